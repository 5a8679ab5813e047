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
// The attention kernel is launched with as many CTAs as the device holds at once.  Its work is cut into
// items (one (b, kv head) column x one run of 256-token tiles); a CTA starts with two items fixed by
// its index and draws the rest from a counter two items ahead, so that the CTAs an SM's schedulers
// favour take more of them.  Staging copies, tile metadata and the query vector of the next tile or
// item are always fetched while the current one is decoded.  When a column has more than one item,
// each leaves a partial result (max, sum, accumulators) and a second kernel merges them.
// Both phases are "decode 128 symbols and dot them with a shared 128-vector", so they share one
// decoder.  The shared vector is held in 16-bit block fixed point (one fp32 step per vector, value
// = step * (256*hi + lo), hi signed and lo unsigned bytes): every table lookup yields up to four
// symbols as four bytes, and two dp4a instructions multiply them with the four matching weight
// bytes -- integer arithmetic, exact, accumulated in int32.  The only rounding is that of the
// weights (2^-16 of the largest weight of the vector); the zero-point terms and everything after
// the dot product are fp32.  With grouped-query attention the G query heads of a KV head share
// every decode: weight records are stored [position][G].
#include <math_constants.h>

#include <mutex>

#include "kvc_decode.cuh"

namespace {

constexpr int SLOT_BYTES = 8192 + 32;     // a block is at most 8191 bytes (u16 fields) + alignment lead
constexpr int SLOT_PAD = 1024;           // readable bytes behind the last staging slot
constexpr int NTHR = 256;
constexpr int ATTN_PART_FLOATS = 4 + 256;   // a partial result of the attention kernel: m, l, two unused, acc[2][128]

struct CacheDev {
    const uint8_t *encoded;
    long long encoded_bytes;
    const uint2 *block_info;
    const uint16_t *thread_info;
    const void *book;
    kvc_qmeta_dev q;
    uint32_t max_block;           // upper bound of a block's byte count
};

CacheDev to_dev(const kvc_cache &c) {
    CacheDev d;
    d.max_block = (c.max_block_bytes > 0 && c.max_block_bytes < 8191) ? (uint32_t)c.max_block_bytes : 8191u;
    d.encoded = c.encoded; d.encoded_bytes = c.encoded_bytes;
    d.block_info = reinterpret_cast<const uint2 *>(c.block_info); d.thread_info = c.thread_info;
    d.book = c.book; d.q = kvc_to_dev(c.q);
    return d;
}

// ---- 16-bit fixed-point weight records -----------------------------------------------------------
// per position c: a word {0, hi(w[c]), hi(w[c+1]), hi(w[c+2])} and a word of the lo bytes laid out the
// same way, so that a decode-table entry {advance, s0, s1, s2} multiplies them directly (the advance
// byte meets the zero).  pack4 gives {hi word, lo word}; q3 is unused.
__device__ __forceinline__ uint2 pack4(int q0, int q1, int q2, int /*q3*/) {
    uint2 r;
    r.x = (((uint32_t)(q0 >> 8) & 0xffu) << 8) | (((uint32_t)(q1 >> 8) & 0xffu) << 16) | (((uint32_t)(q2 >> 8) & 0xffu) << 24);
    r.y = (((uint32_t)q0 & 0xffu) << 8) | (((uint32_t)q1 & 0xffu) << 16) | (((uint32_t)q2 & 0xffu) << 24);
    return r;
}
__device__ __forceinline__ float fix_step(float wmax) { return wmax > 0.f ? wmax * (1.0f / 32767.0f) : 0.f; }
__device__ __forceinline__ int fix_quant(float w, float step) { return step > 0.f ? __float2int_rn(w / step) : 0; }
__device__ __forceinline__ float fix_value(float step, int hi, int lo) { return step * fmaf((float)hi, 256.0f, (float)lo); }

__device__ __forceinline__ uint4 lds128(uint32_t addr) {
    uint4 v;
    asm volatile("ld.shared.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(addr));
    return v;
}

// ---- grouped queries (G >= 2): decode first, multiply afterwards -----------------------------------
// With several query heads per KV head the weight records of a position grow to 16 or 32 bytes, and
// 32 lanes at 32 different positions fetch 0.5-1 KB per lookup: the kernel becomes bound by shared-memory
// wavefronts.  So a thread first decodes its vector into a private row of bytes in shared memory and
// then walks the row four positions at a time; now all lanes of a warp are at the same position, the
// weight words are one broadcast read, and they need no overlapping window: a word holds the hi (or lo)
// bytes of 4 consecutive positions.  The integer sums are the same as in the one-pass form.
constexpr int ROW_STRIDE = 140;           // bytes of a thread's row: 128 symbols + up to 8 of overrun, + 1 word; 35 words spread the banks
static_assert(ROW_STRIDE >= 128 + KVC_DECODE_OVERRUN_PAIR + 3, "rows too short for paired lookups");
constexpr int WROW = 136;                 // weight words per vector of the one-pass form: 128 positions + zeroed overrun
template <int G, bool ROWS> struct VecWords { static constexpr int value = ROWS ? 32 * 2 * G : 2 * WROW * G; };   // weight words of one vector

// {hi word, lo word} of 4 consecutive positions (byte i = position i)
__device__ __forceinline__ uint2 pack4_dense(int q0, int q1, int q2, int q3) {
    uint2 r;
    r.x = ((uint32_t)(q0 >> 8) & 0xffu) | (((uint32_t)(q1 >> 8) & 0xffu) << 8) | (((uint32_t)(q2 >> 8) & 0xffu) << 16) | (((uint32_t)(q3 >> 8) & 0xffu) << 24);
    r.y = ((uint32_t)q0 & 0xffu) | (((uint32_t)q1 & 0xffu) << 8) | (((uint32_t)q2 & 0xffu) << 16) | (((uint32_t)q3 & 0xffu) << 24);
    return r;
}

// decode the thread's vector into `row` (its own 33 words), then dot it with the weight words at w:
// [32 groups of 4 positions][hi | lo][G]
template <int G>
__device__ __forceinline__ bool decode_rows(const uint8_t *slot, uint32_t byte_pos, const KvcBookSmem &book, bool esc,
                                            uint32_t *row, const uint32_t *w, int (&hi)[G], int (&lo)[G]) {
    static_assert(G == 2 || G == 4, "two or four query heads");
    const uint32_t slot_s = kvc_smem_addr(slot), lut_s = kvc_smem_addr(book.lut), tree_s = kvc_smem_addr(book.tree);
    const uint32_t row_s0 = kvc_smem_addr(row);
    // three byte stores per lookup at the position the decoder hands out (its counter starts at the
    // row's address); bytes past the lookup's symbols are rewritten by the next lookup, bytes past
    // position 127 (two lookups per round: up to 8 of them) land in the row's last three words
    auto put = [&](uint32_t e, uint32_t a) {
        asm volatile("st.shared.u8 [%0], %1;\n\tst.shared.u8 [%0+1], %2;\n\tst.shared.u8 [%0+2], %3;"
                     :: "r"(a), "r"(e >> 8), "r"(e >> 16), "r"(e >> 24) : "memory");
    };
    const bool ok = esc ? kvc_decode_vector<true, 0>(slot_s, byte_pos, lut_s, tree_s, row_s0, put)
                        : kvc_decode_vector<false, 0, decltype(put), true>(slot_s, byte_pos, lut_s, tree_s, row_s0, put);
    const uint32_t row_s = kvc_smem_addr(row), w_s = kvc_smem_addr(w);
#pragma unroll 8
    for (int wg = 0; wg < 32; wg++) {
        const uint32_t x = kvc_lds32(row_s + wg * 4);
        if (G == 4) {
            const uint4 a = lds128(w_s + wg * 32), b = lds128(w_s + wg * 32 + 16);
            hi[0] = kvc_dp4a_us(x, a.x, hi[0]); lo[0] = kvc_dp4a_uu(x, b.x, lo[0]);
            hi[1 % G] = kvc_dp4a_us(x, a.y, hi[1 % G]); lo[1 % G] = kvc_dp4a_uu(x, b.y, lo[1 % G]);
            hi[2 % G] = kvc_dp4a_us(x, a.z, hi[2 % G]); lo[2 % G] = kvc_dp4a_uu(x, b.z, lo[2 % G]);
            hi[3 % G] = kvc_dp4a_us(x, a.w, hi[3 % G]); lo[3 % G] = kvc_dp4a_uu(x, b.w, lo[3 % G]);
        } else {
            const uint4 a = lds128(w_s + wg * 16);
            hi[0] = kvc_dp4a_us(x, a.x, hi[0]); lo[0] = kvc_dp4a_uu(x, a.z, lo[0]);
            hi[1 % G] = kvc_dp4a_us(x, a.y, hi[1 % G]); lo[1 % G] = kvc_dp4a_uu(x, a.w, lo[1 % G]);
        }
    }
    return ok;
}

// Where the hi / lo weight word of position c and head g sits in a vector's 2 * WROW * G words.  One or
// two heads: a record {hi[G], lo[G]} per position, fetched with one 8- or 16-byte load.  Four heads: all
// hi records, then all lo records (16 bytes each), because 32-byte records would leave half of the banks idle.
template <int G> __device__ __forceinline__ constexpr int w_hi(int c, int g) { return G == 4 ? c * 4 + g : c * 2 * G + g; }
template <int G> __device__ __forceinline__ constexpr int w_lo(int c, int g) { return G == 4 ? WROW * 4 + c * 4 + g : c * 2 * G + G + g; }

// decode the thread's vector (staged at shared address slot_s) and dot it with the weight records at
// shared address w_s (layout: w_hi / w_lo)
template <int G, bool ESC>
__device__ __forceinline__ bool decode_dot_impl(uint32_t slot_s, uint32_t byte_pos, uint32_t lut_s, uint32_t tree_s,
                                                uint32_t w_s, int (&hi)[G], int (&lo)[G]) {
    constexpr int SHIFT = G == 1 ? 3 : 4;                      // log2 of the record's bytes
    auto emit = [&](uint32_t syms, uint32_t a) {
        if (G == 4) {
            const uint4 x = lds128(a), y = lds128(a + WROW * 16);
            hi[0] = kvc_dp4a_us(syms, x.x, hi[0]); lo[0] = kvc_dp4a_uu(syms, y.x, lo[0]);
            hi[1 % G] = kvc_dp4a_us(syms, x.y, hi[1 % G]); lo[1 % G] = kvc_dp4a_uu(syms, y.y, lo[1 % G]);
            hi[2 % G] = kvc_dp4a_us(syms, x.z, hi[2 % G]); lo[2 % G] = kvc_dp4a_uu(syms, y.z, lo[2 % G]);
            hi[3 % G] = kvc_dp4a_us(syms, x.w, hi[3 % G]); lo[3 % G] = kvc_dp4a_uu(syms, y.w, lo[3 % G]);
        } else if (G == 2) {
            const uint4 x = lds128(a);
            hi[0] = kvc_dp4a_us(syms, x.x, hi[0]); lo[0] = kvc_dp4a_uu(syms, x.z, lo[0]);
            hi[1 % G] = kvc_dp4a_us(syms, x.y, hi[1 % G]); lo[1 % G] = kvc_dp4a_uu(syms, x.w, lo[1 % G]);
        } else {
            const uint2 x = kvc_lds64(a);
            hi[0] = kvc_dp4a_us(syms, x.x, hi[0]);
            lo[0] = kvc_dp4a_uu(syms, x.y, lo[0]);
        }
    };
    // two lookups per round: the weight rows keep WROW - 128 zeroed positions for what is emitted past 127
    static_assert(WROW >= 128 + KVC_DECODE_OVERRUN_PAIR + 1, "weight rows too short for paired lookups");
    return kvc_decode_vector<ESC, SHIFT, decltype(emit), true>(slot_s, byte_pos, lut_s, tree_s, w_s >> SHIFT, emit);
}
// esc: the book has codes longer than the table window (uniform over the CTA)
template <int G>
__device__ __forceinline__ bool decode_dot(const uint8_t *slot, uint32_t byte_pos, const KvcBookSmem &book, bool esc,
                                           const uint32_t *w, int (&hi)[G], int (&lo)[G]) {
    const uint32_t slot_s = kvc_smem_addr(slot), lut_s = kvc_smem_addr(book.lut), tree_s = kvc_smem_addr(book.tree),
                   w_s = kvc_smem_addr(w);
    return esc ? decode_dot_impl<G, true>(slot_s, byte_pos, lut_s, tree_s, w_s, hi, lo)
               : decode_dot_impl<G, false>(slot_s, byte_pos, lut_s, tree_s, w_s, hi, lo);
}
__device__ __forceinline__ bool book_has_long_codes(const void *book) {
    return kvc_book_needs_escape(book);
}

// ---- staging --------------------------------------------------------------------------------------
// plain loads: the 64 threads of a sub-group copy block `blk` into `slot`
// *nb receives the block's byte count: a vector that starts at or beyond it is not decoded
__device__ __forceinline__ bool stage(const CacheDev &kc, long long blk, uint8_t *slot, uint32_t *lead, uint32_t *nb, int v) {
    const uint2 bi = kc.block_info[blk];
    const uint32_t nbytes = bi.y & 0xffffu;
    *nb = nbytes;
    if (nbytes == 0 || nbytes > kc.max_block || (long long)bi.x + nbytes > kc.encoded_bytes) { *lead = 0; *nb = 0; return false; }
    *lead = kvc_stage_block(slot, kc.encoded, kc.encoded_bytes, bi.x, nbytes, v, 64);
    return true;
}

// bulk copies: lane `l` (< 4) of one warp issues the copy of its block; the whole warp must call.
// The source range is widened to 16-byte boundaries; `encoded` is 16-byte aligned and readable to
// the next boundary past its end (checked / required by the host code).
// starve (tests of the bounded waits only): announce 16 bytes and copy nothing, so that the phase never
// completes and nothing is in flight when the waiting threads give up.
__device__ __forceinline__ void stage_bulk(const CacheDev &kc, bool valid, long long blk, uint8_t *slot,
                                           uint32_t *lead, int *ok, uint32_t *nb, uint64_t *bar, int lane, bool starve = false) {
    uint32_t bytes = 0, ld = 0, nbytes = 0;
    const uint8_t *a0 = nullptr;
    bool good = false;
    if (lane < 4 && valid) {
        const uint2 bi = kc.block_info[blk];
        nbytes = bi.y & 0xffffu;
        good = nbytes != 0 && nbytes <= kc.max_block && (long long)bi.x + nbytes <= kc.encoded_bytes;
        if (good) {
            const uint8_t *src = kc.encoded + bi.x;
            ld = (uint32_t)(reinterpret_cast<uintptr_t>(src) & 15);
            a0 = src - ld;
            bytes = (ld + nbytes + 15u) & ~15u;
        }
    }
    if (starve) bytes = 0;
    uint32_t total = bytes;
    total += __shfl_xor_sync(0xffffffffu, total, 1);
    total += __shfl_xor_sync(0xffffffffu, total, 2);
    if (lane == 0) kvc_mbar_expect_tx(bar, starve ? 16u : total);   // one arrival per phase, even for 0 bytes
    __syncwarp();
    if (lane < 4) {
        lead[lane] = ld; ok[lane] = good; nb[lane] = good ? nbytes : 0u;
        if (bytes) kvc_bulk_g2s(slot, a0, bytes, bar);
    }
}

__device__ __forceinline__ uint32_t vec_start(const uint16_t *thread_info, long long blk, int v) {
    return v ? (uint32_t)(thread_info[blk * 64 + v - 1] >> 3) : 0u;
}
// the same in two steps: the load (issued a tile ahead) and the shift (at the use)
__device__ __forceinline__ unsigned short vec_start_bits(const uint16_t *thread_info, long long blk, int v) {
    unsigned short r = 0;
    if (v) r = thread_info[blk * 64 + v - 1];
    return r;
}

// ---- K weights --------------------------------------------------------------------------------------
// Weight records of the 4 blocks of a 256-token tile: w[sub][c][hi|lo][g], step[sub][g], zp[sub][g].
// Warp `wp` owns block sub = wp & 3 and the query heads g = (wp >> 2) * GH .. + GH - 1 (GH = G/2, or
// all of them on warps 0-3 when G = 1); lane = 4 consecutive channels.
// Units that depend on the channel (sc != 0) need tok_div % 64 == 0 so that a block shares them;
// otherwise scale and min_int are per-token scalars applied after the dot product (k_finish).
// scale (fp16 bits) and min_int of the lane's 4 consecutive channels, as two vector loads leave them: no
// arithmetic touches the words before their use, and they occupy 3 or 4 registers instead of 8
struct KUnit { uint2 sc; uint2 mi; };
__device__ __forceinline__ unsigned short ku_scale(const KUnit &u, int i) {
    const uint32_t w = i < 2 ? u.sc.x : u.sc.y;
    return (unsigned short)((i & 1) ? (w >> 16) : (w & 0xffffu));
}
__device__ __forceinline__ int ku_min(const KUnit &u, int i, int min_bytes) {
    if (min_bytes == 1) return (int)(signed char)((u.mi.x >> (8 * i)) & 0xffu);
    const uint32_t w = i < 2 ? u.mi.x : u.mi.y;
    return (int)(short)((i & 1) ? (w >> 16) : (w & 0xffffu));
}

// global -> registers; issued a tile ahead so that the latency hides behind the decode
__device__ __forceinline__ void k_units_load(KUnit &u, const kvc_qmeta_dev &m, long long tok0, long long T,
                                             long long b, long long h, int tid) {
    const int lane = tid & 31, sub = (tid >> 5) & 3;
    const long long t = tok0 + sub * 64;
    u.sc = make_uint2(0x3c003c00u, 0x3c003c00u); u.mi = make_uint2(0u, 0u);          // 1.0, 0
    if (m.sc != 0 && t < T) {                              // channel units lie side by side (sc == 1, checked by the host)
        const long long un = kvc_tok_unit(t, m.tok_div) * m.sj + b * m.sb + h * m.sh + lane * 4;
        u.sc = *reinterpret_cast<const uint2 *>(reinterpret_cast<const unsigned short *>(m.scale) + un);
        if (m.min_bytes == 1) u.mi.x = *reinterpret_cast<const uint32_t *>(reinterpret_cast<const int8_t *>(m.min_int) + un);
        else u.mi = *reinterpret_cast<const uint2 *>(reinterpret_cast<const int16_t *>(m.min_int) + un);
    }
}

// ROWS: the layout of decode_rows (grouped queries in the attention kernel) instead of w_hi / w_lo
template <int G, bool ROWS = false>
__device__ __forceinline__ void k_weights_build(uint32_t *w, float *step, float *zp, const float *qf, const KUnit &u,
                                                bool channel_units, int min_bytes, long long tok0, long long T, int tid) {
    const int lane = tid & 31, wp = tid >> 5, sub = wp & 3;
    constexpr int GH = G >= 2 ? G / 2 : 1;
    if (G == 1 && wp >= 4) return;
    const bool live = tok0 + sub * 64 < T;
#pragma unroll
    for (int gi = 0; gi < GH; gi++) {
        const int g = G == 1 ? 0 : (wp >> 2) * GH + gi;
        float wv[4], z = 0.f;
#pragma unroll
        for (int i = 0; i < 4; i++) {
            const float q = live ? qf[g * 128 + lane * 4 + i] : 0.f;
            const float sc = kvc_scale_value(ku_scale(u, i));
            wv[i] = q * sc;
            z = fmaf((float)ku_min(u, i, min_bytes) * sc, q, z);
        }
        float mx = fmaxf(fmaxf(fabsf(wv[0]), fabsf(wv[1])), fmaxf(fabsf(wv[2]), fabsf(wv[3])));
        mx = kvc_warp_max(mx);
        z = channel_units ? kvc_warp_sum(z) : 0.f;
        const float st = fix_step(mx), inv = st > 0.f ? 1.0f / st : 0.f;
        int q4[7];
#pragma unroll
        for (int i = 0; i < 4; i++) q4[i] = __float2int_rn(wv[i] * inv);
        uint32_t *row = w + (size_t)sub * VecWords<G, ROWS>::value;
        if (ROWS) {                                             // the lane's 4 positions are one group: [group][hi | lo][g]
            const uint2 r = pack4_dense(q4[0], q4[1], q4[2], q4[3]);
            row[(lane * 2 + 0) * G + g] = r.x; row[(lane * 2 + 1) * G + g] = r.y;
        } else {
#pragma unroll
            for (int i = 0; i < 3; i++) {                       // the next lane's first three values
                int nv = __shfl_down_sync(0xffffffffu, q4[i], 1);
                q4[4 + i] = lane == 31 ? 0 : nv;
            }
#pragma unroll
            for (int i = 0; i < 4; i++) {                       // layout: w_hi / w_lo
                const uint2 r = pack4(q4[i], q4[i + 1], q4[i + 2], q4[i + 3]);
                row[w_hi<G>(lane * 4 + i, g)] = r.x; row[w_lo<G>(lane * 4 + i, g)] = r.y;
            }
            if (lane < WROW - 128) { row[w_hi<G>(128 + lane, g)] = 0u; row[w_lo<G>(128 + lane, g)] = 0u; }
        }
        if (lane == 0) { step[sub * G + g] = st; zp[sub * G + g] = z; }
    }
}

template <int G>
__device__ __forceinline__ void k_weights(uint32_t *w, float *step, float *zp, const float *qf, const kvc_qmeta_dev &m,
                                          long long tok0, long long T, long long b, long long h, int tid) {
    KUnit u;
    k_units_load(u, m, tok0, T, b, h, tid);
    k_weights_build<G>(w, step, zp, qf, u, m.sc != 0, m.min_bytes, tok0, T, tid);
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

// scale and min_int of a token whose K units do not depend on the channel (loaded ahead of the decode)
__device__ __forceinline__ void k_token_unit(unsigned short &sc, int &mi, const kvc_qmeta_dev &m, long long t,
                                             long long b, long long h) {
    const long long u = kvc_tok_unit(t, m.tok_div) * m.sj + b * m.sb + h * m.sh;
    sc = kvc_load_scale_bits(m, u); mi = kvc_load_min(m, u);
}

// sum of each query head's 128 (scaled) values: one warp per head; needs a barrier before and after
template <int G>
__device__ __forceinline__ void q_sums(const float *qf, float *qsum, int tid) {
    if (tid < G * 32) {
        const int g = tid >> 5, lane = tid & 31;
        float s = qf[g * 128 + lane] + qf[g * 128 + lane + 32] + qf[g * 128 + lane + 64] + qf[g * 128 + lane + 96];
        s = kvc_warp_sum(s);
        if (lane == 0) qsum[g] = s;
    }
}

// score of the thread's token from its integer dot products
template <int G>
__device__ __forceinline__ void k_finish(float (&s)[G], const int (&hi)[G], const int (&lo)[G], const float *step_sub,
                                         const float *zp_sub, const float *qsum, bool channel_units, float sc, float mi) {
#pragma unroll
    for (int g = 0; g < G; g++) {
        const float d = fix_value(step_sub[g], hi[g], lo[g]);
        s[g] = channel_units ? d + zp_sub[g] : sc * fmaf(mi, qsum[g], d);
    }
}

// ---- V weights --------------------------------------------------------------------------------------
// Called by all 256 threads (thread = token of the tile, grp = its 128-token group, tl = its index in
// the group) with wv[g] = p[g] * scale of the token.  Builds records ps[grp][tl][hi|lo][g], step[grp][g].
// `red` is scratch for 8*G floats, `q16` for 2*G*(128+4) int16 (unused with ROWS).  Contains three block
// barriers (two with ROWS).
template <int G, bool ROWS = false>
__device__ __forceinline__ void v_weights(uint32_t *ps, float *vstep, float *red, int16_t *q16, const float (&wv)[G],
                                          int tid) {
    const int lane = tid & 31, warp = tid >> 5, grp = tid >> 7, tl = tid & 127;
#pragma unroll
    for (int g = 0; g < G; g++) { float mx = kvc_warp_max(fabsf(wv[g])); if (lane == 0) red[warp * G + g] = mx; }
    if (!ROWS && tl < 4) for (int g = 0; g < G; g++) q16[(grp * G + g) * 132 + 128 + tl] = 0;
    __syncthreads();
    if (ROWS) {
        // four consecutive tokens make one weight word per head: their 16-bit values reach the first of
        // the four lanes by shuffles, no scratch and no barrier in between
#pragma unroll
        for (int g = 0; g < G; g++) {
            const float mx = fmaxf(fmaxf(red[(grp * 4 + 0) * G + g], red[(grp * 4 + 1) * G + g]),
                                   fmaxf(red[(grp * 4 + 2) * G + g], red[(grp * 4 + 3) * G + g]));
            const float st = fix_step(mx);
            const int q0 = fix_quant(wv[g], st);
            const int q1 = __shfl_down_sync(0xffffffffu, q0, 1), q2 = __shfl_down_sync(0xffffffffu, q0, 2),
                      q3 = __shfl_down_sync(0xffffffffu, q0, 3);
            if (tl == 0) vstep[grp * G + g] = st;
            if ((tl & 3) == 0) {                               // [group of 4 tokens][hi | lo][g]
                uint32_t *row = ps + (size_t)grp * VecWords<G, ROWS>::value;
                const uint2 r = pack4_dense(q0, q1, q2, q3);
                row[((tl >> 2) * 2 + 0) * G + g] = r.x; row[((tl >> 2) * 2 + 1) * G + g] = r.y;
            }
        }
        __syncthreads();
        return;
    }
#pragma unroll
    for (int g = 0; g < G; g++) {
        const float mx = fmaxf(fmaxf(red[(grp * 4 + 0) * G + g], red[(grp * 4 + 1) * G + g]),
                               fmaxf(red[(grp * 4 + 2) * G + g], red[(grp * 4 + 3) * G + g]));
        const float st = fix_step(mx);
        q16[(grp * G + g) * 132 + tl] = (int16_t)fix_quant(wv[g], st);
        if (tl == 0) vstep[grp * G + g] = st;
    }
    __syncthreads();
#pragma unroll
    for (int g = 0; g < G; g++) {
        const int16_t *qq = q16 + (grp * G + g) * 132 + tl;
        uint32_t *row = ps + (size_t)grp * VecWords<G, ROWS>::value;    // layout: w_hi / w_lo
        const uint2 r = pack4(qq[0], qq[1], qq[2], qq[3]);
        row[w_hi<G>(tl, g)] = r.x; row[w_lo<G>(tl, g)] = r.y;
        if (tl < WROW - 128) { row[w_hi<G>(128 + tl, g)] = 0u; row[w_lo<G>(128 + tl, g)] = 0u; }
    }
    __syncthreads();
}

// ---- fused K: raw scores ------------------------------------------------------------------------
template <int G>
struct QkSmem {
    KvcBookSmem book;
    uint8_t slot[4][SLOT_BYTES];
    alignas(32) uint32_t w[4 * 2 * WROW * G];
    float step[4 * G];
    float zp[4 * G];
    float qf[G * 128];
    float qsum[G];
    uint32_t lead[4], nb[4];
    int ok[4];
};

template <int G>
__global__ void __launch_bounds__(NTHR) fused_qk_kernel(CacheDev kc, long long T, long long B, long long Hkv, long long Hq,
                                                        long long g0, const __half *__restrict__ q, void *__restrict__ out,
                                                        int out_f32, int *__restrict__ status) {
    extern __shared__ __align__(128) uint8_t smem_raw[];
    QkSmem<G> &sm = *reinterpret_cast<QkSmem<G> *>(smem_raw);
    const int tid = threadIdx.x, sub = tid >> 6, v = tid & 63;
    const long long cols = B * Hkv, col = blockIdx.y, b = col / Hkv, h = col % Hkv;
    const long long Gt = Hq / Hkv, hq0 = h * Gt + g0;
    const long long tok0 = (long long)blockIdx.x * 256, t = tok0 + tid;
    kvc_load_book(sm.book, kc.book, tid, NTHR);
    const bool esc = book_has_long_codes(kc.book);
    load_q<G>(sm.qf, sm.qsum, q, b, Hq, hq0, 1.0f, tid);
    const long long blk = (tok0 / 64 + sub) * cols + col;
    const bool active = t < T;
    if (active) { uint32_t ld, nb; bool ok = stage(kc, blk, sm.slot[sub], &ld, &nb, v); if (v == 0) { sm.lead[sub] = ld; sm.nb[sub] = nb; sm.ok[sub] = ok; } }
    __syncthreads();
    k_weights<G>(sm.w, sm.step, sm.zp, sm.qf, kc.q, tok0, T, b, h, tid);
    __syncthreads();
    if (!active) return;
    unsigned short ksc = 0x3c00; int kmi = 0;
    if (kc.q.sc == 0) k_token_unit(ksc, kmi, kc.q, t, b, h);
    int hi[G], lo[G];
#pragma unroll
    for (int g = 0; g < G; g++) { hi[g] = 0; lo[g] = 0; }
    const uint32_t start = vec_start(kc.thread_info, blk, v);
    bool ok = sm.ok[sub] && start < sm.nb[sub];                // a vector begins inside its block
    if (ok) ok = decode_dot<G>(sm.slot[sub], sm.lead[sub] + start, sm.book, esc, sm.w + sub * 2 * WROW * G, hi, lo);
    if (!ok) atomicOr(status, KVC_FLAG_BAD_STREAM);
    float s[G];
    k_finish<G>(s, hi, lo, sm.step + sub * G, sm.zp + sub * G, sm.qsum, kc.q.sc != 0, kvc_scale_value(ksc), (float)kmi);
#pragma unroll
    for (int g = 0; g < G; g++) {
        const long long o = (b * Hq + hq0 + g) * T + t;
        if (out_f32) reinterpret_cast<float *>(out)[o] = s[g];
        else reinterpret_cast<__half *>(out)[o] = __float2half_rn(s[g]);
    }
}

// ---- fused V: per-group partial outputs ----------------------------------------------------------
template <int G>
struct PvSmem {
    KvcBookSmem book;
    uint8_t slot[4][SLOT_BYTES];
    alignas(32) uint32_t ps[2 * 2 * WROW * G];
    float vstep[2 * G];
    float zpv[2 * G];
    float red[2][8 * G];
    int16_t q16[2 * G * 132];
    uint32_t lead[4], nb[4];
    int ok[4];
};

template <int G>
__global__ void __launch_bounds__(NTHR) fused_pv_kernel(CacheDev vc, long long T, long long B, long long Hkv, long long Hq,
                                                        long long g0, const __half *__restrict__ P, __half *__restrict__ out,
                                                        int *__restrict__ status) {
    extern __shared__ __align__(128) uint8_t smem_raw[];
    PvSmem<G> &sm = *reinterpret_cast<PvSmem<G> *>(smem_raw);
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, sub = tid >> 6, v = tid & 63;
    const int grp = tid >> 7, ch = tid & 127;
    const long long cols = B * Hkv, col = blockIdx.y, b = col / Hkv, h = col % Hkv;
    const long long Gt = Hq / Hkv, hq0 = h * Gt + g0;
    const long long tok0 = (long long)blockIdx.x * 256, t = tok0 + tid;
    const kvc_qmeta_dev &m = vc.q;
    kvc_load_book(sm.book, vc.book, tid, NTHR);
    const bool esc = book_has_long_codes(vc.book);
    const long long gI = tok0 / 128 + grp;
    const long long blk = gI * (cols * 2) + col * 2 + (ch >> 6);
    const bool active = gI * 128 < T;
    if (active) { uint32_t ld, nb; bool ok = stage(vc, blk, sm.slot[sub], &ld, &nb, v); if (v == 0) { sm.lead[sub] = ld; sm.nb[sub] = nb; sm.ok[sub] = ok; } }
    float wv[G];
    {
        float sc = 0.f, mi = 0.f;
        if (t < T) {
            const long long u = kvc_tok_unit(t, m.tok_div) * m.sj + b * m.sb + h * m.sh;
            sc = __half2float(m.scale[u]); mi = (float)kvc_load_min(m, u);
        }
#pragma unroll
        for (int g = 0; g < G; g++) {
            const float p = t < T ? __half2float(P[(b * Hq + hq0 + g) * T + t]) : 0.f;
            wv[g] = p * sc;
            const float z = kvc_warp_sum(wv[g] * mi);
            if (lane == 0) sm.red[1][warp * G + g] = z;
        }
    }
    v_weights<G>(sm.ps, sm.vstep, sm.red[0], sm.q16, wv, tid);
    if (!active) return;
    int hi[G], lo[G];
#pragma unroll
    for (int g = 0; g < G; g++) { hi[g] = 0; lo[g] = 0; }
    const uint32_t start = vec_start(vc.thread_info, blk, v);
    bool ok = sm.ok[sub] && start < sm.nb[sub];
    if (ok) ok = decode_dot<G>(sm.slot[sub], sm.lead[sub] + start, sm.book, esc, sm.ps + grp * 2 * WROW * G, hi, lo);
    if (!ok) atomicOr(status, KVC_FLAG_BAD_STREAM);
#pragma unroll
    for (int g = 0; g < G; g++) {
        const float z = sm.red[1][(grp * 4 + 0) * G + g] + sm.red[1][(grp * 4 + 1) * G + g] +
                        sm.red[1][(grp * 4 + 2) * G + g] + sm.red[1][(grp * 4 + 3) * G + g];
        out[((gI * B + b) * Hq + hq0 + g) * 128 + ch] = __float2half_rn(fix_value(sm.vstep[grp * G + g], hi[g], lo[g]) + z);
    }
}

// ---- one-pass decode attention -------------------------------------------------------------------
template <int G>
struct alignas(32) AttnSmem {                     // followed in shared memory by 4 K slots, 4 V slots (sized at launch),
    KvcBookSmem bookK, bookV;         // SLOT_PAD bytes that a corrupt stream's decoder overrun may read
    alignas(32) uint32_t w[4 * VecWords<G, (G >= 2)>::value];     // K weight words; reused by v_weights (scratch), the tail and the final cross-group sum
    alignas(32) uint32_t ps[2 * VecWords<G, (G >= 2)>::value];    // V weight words
    float kstep[4 * G], zp[4 * G];
    float vstep[2 * G];
    float qf[G * 128];
    float qsum[G];
    float red[4][8 * G];              // per-warp max, sum, zpv and weight-max partials
    uint64_t bar[2];                  // K and V staging barriers
    uint32_t leadK[4], leadV[4];
    uint32_t nbK[4], nbV[4];          // byte counts of the staged blocks
    int okK[4], okV[4];
    int next_j;                       // item the CTA drew for after the current one
    int dead;                         // a staging wait ran out: the CTA takes no further item
};

struct AttnParams {
    CacheDev k, v;
    long long T, B, Hkv, Hq, g0, Tr;
    const __half *q, *ktail, *vtail;
    __half *out;
    float scaling;
    int n_tiles;                  // 256-token tiles per column
    // every column is cut into `long_runs` runs of `tiles_per_split` tiles followed by `splits - long_runs`
    // runs of `short_tiles` tiles; the items of the long runs of all columns come first, the short ones last
    int splits, tiles_per_split, long_runs, short_tiles;
    long long work;               // columns * splits items
    uint32_t slotK_bytes, slotV_bytes;   // capacity of one staging slot (multiple of 16)
    float *ws_part;               // [B*Hq][splits][ATTN_PART_FLOATS]
    int *sched;                   // {items handed out, CTAs finished}, or null: static shares
    int *status;
    int partial;                  // items leave partial results for the merge kernel (several runs per column, or a tail that the merge kernel adds)
    int wait_limit;               // tries of a staging wait before it gives up (KVC_FLAG_WAIT_TIMEOUT)
    int starve;                   // tests of the bounded waits only: announce bytes that are never copied
};

// BULK: stage with bulk asynchronous copies (one tile phase ahead) instead of plain loads.
template <int G, bool BULK>
__global__ void __launch_bounds__(NTHR, G == 4 ? 2 : 3) attn_decode_kernel(AttnParams p) {
    extern __shared__ __align__(128) uint8_t smem_raw[];
    AttnSmem<G> &sm = *reinterpret_cast<AttnSmem<G> *>(smem_raw);
    uint8_t *const slotsK = smem_raw + sizeof(AttnSmem<G>), *const slotsV = slotsK + 4 * p.slotK_bytes;
    constexpr bool ROWS = G >= 2;                          // grouped queries: decode into rows, multiply afterwards
    uint32_t *const myrow = reinterpret_cast<uint32_t *>(slotsV + 4 * p.slotV_bytes + SLOT_PAD) + threadIdx.x * (ROW_STRIDE / 4);
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, sub = tid >> 6, v = tid & 63;
    const int grp = tid >> 7, ch = tid & 127;
    // Launched with programmatic stream serialisation.  This kernel's own set-up -- the books' tables, the first
    // blocks, the first tile's metadata: cache data that no kernel of a decode step writes -- runs before
    // griddepcontrol.wait, i.e. possibly while the kernel ahead of it in the stream (the merge of the layer
    // before, which lets its dependents start early) still runs.  What that kernel or the one before it may
    // write (the query, the scheduling counters, the workspace, the output, the status word) is touched after
    // the wait.  (Letting this kernel's own dependents start early was measured: their waiting CTAs slow the
    // launch by a tenth.)
    // shapes fit 32 bits (the host checks): 64-bit arithmetic only where block ids and addresses are formed
    const int T = (int)p.T, B = (int)p.B, Hkv = (int)p.Hkv, Hq = (int)p.Hq;
    const int cols = B * Hkv, Gt = Hq / Hkv;
    const int n_tiles = p.n_tiles;
    const kvc_qmeta_dev &km = p.k.q, &vm = p.v.q;
    int flags = 0;

    // The work is cut into items: a column (one sequence, one KV head) x one of `splits` runs of
    // `tiles_per_split` tiles; item j = column * splits + run.  Without a scheduling counter CTA i of P
    // takes the items [work*i/P, work*(i+1)/P).  With one it takes items i and P + i and draws every
    // further item from the counter, two items ahead of its use so that the answer has an item's time
    // to arrive: CTAs that run faster (the warp schedulers favour some of an SM's CTAs) take more.
    struct Item { int col, t_lo, t_hi, part; };            // part: the run's index within its column
    const bool draw = p.sched != nullptr;
    const int P = (int)gridDim.x;                           // items are counted in 32 bits (the host checks the range)
    const int w_hi = draw ? (int)p.work : (int)(p.work * (blockIdx.x + 1) / P);
    auto item_of = [&](int j, Item &it) -> bool {
        if (j >= w_hi) return false;
        const int n_long = (int)cols * p.long_runs;          // items of long runs; the short runs follow: the last
        if (j < n_long) {                                    // items to be drawn are short, so the CTAs end close together
            const int r = j % p.long_runs;
            it.col = j / p.long_runs; it.part = r; it.t_lo = r * p.tiles_per_split; it.t_hi = min(n_tiles, it.t_lo + p.tiles_per_split);
        } else {
            const int n_short = p.splits - p.long_runs, r = (j - n_long) % n_short;
            it.col = (j - n_long) / n_short; it.part = p.long_runs + r;
            it.t_lo = p.long_runs * p.tiles_per_split + r * p.short_tiles; it.t_hi = min(n_tiles, it.t_lo + p.short_tiles);
        }
        return true;
    };

    // block ids of a tile's four K blocks / four V blocks for lane l < 4 of the issuing warp
    auto blkK_of = [&](int col, int tile, int l) { return ((long long)tile * 4 + l) * cols + col; };
    auto blkV_of = [&](int col, int tile, int l) { return ((long long)tile * 2 + (l >> 1)) * (cols * 2) + (long long)col * 2 + (l & 1); };
    auto validK = [&](bool on, int tile, int l) { return on && (long long)tile * 256 + l * 64 < T; };
    auto validV = [&](bool on, int tile, int l) { return on && (long long)tile * 256 + (l >> 1) * 128 < T; };

    Item it, nit;
    int j_it = draw ? (int)blockIdx.x : (int)(p.work * blockIdx.x / P), j_n1 = draw ? P + (int)blockIdx.x : j_it + 1;
    bool have = item_of(j_it, it), have_next = have && item_of(j_n1, nit);
    int drawn = 0;                                         // thread 0: the counter's answer, used an item later
    const bool any_tiles = have && it.t_lo < it.t_hi;      // items are empty only when the cache has no compressed part

    if (BULK) {
        if (tid == 0) { kvc_mbar_init(&sm.bar[0], 1); kvc_mbar_init(&sm.bar[1], 1); kvc_mbar_fence_init(); sm.dead = 0; }
        __syncthreads();
        if (warp == 0 && any_tiles) {
            stage_bulk(p.k, validK(true, it.t_lo, lane & 3), blkK_of(it.col, it.t_lo, lane & 3), slotsK + (lane & 3) * p.slotK_bytes, sm.leadK, sm.okK, sm.nbK, &sm.bar[0], lane, p.starve != 0);
            stage_bulk(p.v, validV(true, it.t_lo, lane & 3), blkV_of(it.col, it.t_lo, lane & 3), slotsV + (lane & 3) * p.slotV_bytes, sm.leadV, sm.okV, sm.nbV, &sm.bar[1], lane, p.starve != 0);
        }
    }
    bool escK = false, escV = false;
    if (p.T > 0) {                                         // (no streams at all while nothing is compressed yet)
        kvc_load_book(sm.bookK, p.k.book, tid, NTHR);
        kvc_load_book(sm.bookV, p.v.book, tid, NTHR);
        escK = book_has_long_codes(p.k.book); escV = book_has_long_codes(p.v.book);
    }

    // Per-thread metadata of a tile (vector start offsets, the token's V scale / min_int, the K unit
    // parameters of the warp's block) is fetched one tile ahead, so that no global-memory latency
    // sits between the phases of a tile.
    struct TileMeta { unsigned short startK, startV, vsc, ksc; int vmi, kmi; KUnit ku; };   // as loaded: no arithmetic waits on them here
    auto load_meta = [&](bool on, int col, int tile, TileMeta &tm) {
        const long long tok0 = (long long)tile * 256, t = tok0 + tid;
        const long long gI = tok0 / 128 + grp;
        const int b = col / (int)Hkv, h = col % (int)Hkv;
        tm.startK = tm.startV = 0; tm.vsc = 0; tm.vmi = tm.kmi = 0; tm.ksc = 0x3c00;
        if (on) {
            if (t < T) {
                tm.startK = vec_start_bits(p.k.thread_info, (tok0 / 64 + sub) * cols + col, v);
                const long long u = kvc_tok_unit(t, vm.tok_div) * vm.sj + b * vm.sb + h * vm.sh;
                tm.vsc = kvc_load_scale_bits(vm, u); tm.vmi = kvc_load_min(vm, u);
                if (km.sc == 0) k_token_unit(tm.ksc, tm.kmi, km, t, b, h);
            }
            if (gI * 128 < T) tm.startV = vec_start_bits(p.v.thread_info, gI * (cols * 2) + (long long)col * 2 + (ch >> 6), v);
        }
        k_units_load(tm.ku, km, on ? tok0 : T, T, b, h, tid);
    };
    TileMeta cur, nxt;
    load_meta(any_tiles, have ? it.col : 0, have ? it.t_lo : 0, cur);

    // The query values of an item are fetched (as fp16 bits) while the item before it still runs.
    constexpr int QN = (G * 128 + NTHR - 1) / NTHR;
    unsigned short qn[QN];
    auto q_fetch = [&](int col_) {
        const long long row0 = (long long)(col_ / (int)Hkv) * Hq + (long long)(col_ % (int)Hkv) * Gt + p.g0;
#pragma unroll
        for (int i = 0; i < QN; i++) {
            const int idx = tid + i * NTHR;
            qn[i] = 0;
            if (idx < G * 128) qn[i] = reinterpret_cast<const unsigned short *>(p.q)[(row0 + (idx >> 7)) * 128 + (idx & 127)];
        }
    };
    auto q_store = [&]() {
#pragma unroll
        for (int i = 0; i < QN; i++) {
            const int idx = tid + i * NTHR;
            if (idx < G * 128) sm.qf[idx] = kvc_scale_value(qn[i]) * p.scaling;
        }
    };
    asm volatile("griddepcontrol.wait;" ::: "memory");
    if (have) q_fetch(it.col);

    uint32_t par = 0;                                      // bit 0 / bit 1: parity of the staging phase the K / V barrier is waited for next
    while (have) {
    const int col = it.col, b = col / (int)Hkv, h = col % (int)Hkv;
    const long long hq0 = h * Gt + p.g0;
    if (draw && tid == 0) drawn = atomicAdd(&p.sched[0], 1);
    q_store();                                             // fetched during the previous item's last tile
    __syncthreads();
    q_sums<G>(sm.qf, sm.qsum, tid);
    __syncthreads();                                       // books, q and (unbuffered) slots are in place
    float m_run[G], l_run[G], acc[G];
#pragma unroll
    for (int g = 0; g < G; g++) { m_run[g] = -CUDART_INF_F; l_run[g] = 0.f; acc[g] = 0.f; }

    for (int tile = it.t_lo; tile < it.t_hi; tile++) {
        const long long tok0 = (long long)tile * 256, t = tok0 + tid;
        const long long blkK = (tok0 / 64 + sub) * cols + col;
        const long long gI = tok0 / 128 + grp;
        const long long blkV = gI * (cols * 2) + (long long)col * 2 + (ch >> 6);
        const bool actK = t < T, actV = gI * 128 < T;
        // the tile after this one in the CTA's sequence (it may open the next column)
        bool n_on = true; int n_col = col, n_tile = tile + 1;
        if (n_tile >= it.t_hi) {
            n_on = have_next && nit.t_lo < nit.t_hi; n_col = n_on ? nit.col : col; n_tile = n_on ? nit.t_lo : 0;
            if (have_next) q_fetch(nit.col);
        }
        if (!BULK) {
            if (actK) { uint32_t ld, nb; bool ok = stage(p.k, blkK, slotsK + sub * p.slotK_bytes, &ld, &nb, v); if (v == 0) { sm.leadK[sub] = ld; sm.nbK[sub] = nb; sm.okK[sub] = ok; } }
            if (actV) { uint32_t ld, nb; bool ok = stage(p.v, blkV, slotsV + sub * p.slotV_bytes, &ld, &nb, v); if (v == 0) { sm.leadV[sub] = ld; sm.nbV[sub] = nb; sm.okV[sub] = ok; } }
        }
        k_weights_build<G, ROWS>(sm.w, sm.kstep, sm.zp, sm.qf, cur.ku, km.sc != 0, km.min_bytes, tok0, T, tid);
        // A wait that runs out: the thread does not decode.  The warp that issues the copies looks at its own
        // verdict: a barrier whose phase it did not see complete is never armed again (a second arrival on an
        // open phase is an error), and the CTA is marked; it takes no further item, and what it had in flight
        // is waited for once more, bounded, before it returns.
        bool k_landed = true;
        if (BULK) {
            k_landed = kvc_mbar_wait(&sm.bar[0], par & 1u, p.wait_limit);
            if (k_landed) par ^= 1u; else flags |= KVC_FLAG_WAIT_TIMEOUT;
        }
        __syncthreads();
        // ---- K: scores of this tile's tokens
        float s[G];
        if (actK) {
            int hi[G], lo[G];
#pragma unroll
            for (int g = 0; g < G; g++) { hi[g] = 0; lo[g] = 0; }
            bool ok = k_landed && sm.okK[sub] && (uint32_t)(cur.startK >> 3) < sm.nbK[sub];      // a vector begins inside its block
            if (ok) {
                if constexpr (ROWS) ok = decode_rows<G>(slotsK + sub * p.slotK_bytes, sm.leadK[sub] + (cur.startK >> 3), sm.bookK, escK, myrow, sm.w + sub * VecWords<G, true>::value, hi, lo);
                else ok = decode_dot<G>(slotsK + sub * p.slotK_bytes, sm.leadK[sub] + (cur.startK >> 3), sm.bookK, escK, sm.w + sub * VecWords<G, false>::value, hi, lo);
            }
            if (!ok) flags |= KVC_FLAG_BAD_STREAM;
            k_finish<G>(s, hi, lo, sm.kstep + sub * G, sm.zp + sub * G, sm.qsum, km.sc != 0, kvc_scale_value(cur.ksc), (float)cur.kmi);
        } else {
#pragma unroll
            for (int g = 0; g < G; g++) s[g] = -CUDART_INF_F;
        }
        // ---- online softmax over the tile
#pragma unroll
        for (int g = 0; g < G; g++) { float mx = kvc_warp_max(s[g]); if (lane == 0) sm.red[0][warp * G + g] = mx; }
        __syncthreads();                                   // also: every thread is done with the K slots
        // the next tile's per-thread metadata is asked for now and first touched when that tile begins: it is in
        // flight during the V phase only, and the K decode above ran without its registers
        load_meta(n_on, n_col, n_tile, nxt);
        if (BULK && warp == 0) {                           // next tile's K blocks land during the V phase
            if (__all_sync(0xffffffffu, k_landed))
                stage_bulk(p.k, validK(n_on, n_tile, lane & 3), blkK_of(n_col, n_tile, lane & 3), slotsK + (lane & 3) * p.slotK_bytes, sm.leadK, sm.okK, sm.nbK, &sm.bar[0], lane, p.starve != 0);
            else if (lane == 0) sm.dead = 1;
        }
        float alpha[G], wv[G];
#pragma unroll
        for (int g = 0; g < G; g++) {
            float mt = sm.red[0][g];
#pragma unroll
            for (int w8 = 1; w8 < 8; w8++) mt = fmaxf(mt, sm.red[0][w8 * G + g]);
            const float m_new = fmaxf(m_run[g], mt);
            alpha[g] = __expf(m_run[g] - m_new);           // exp(-inf) = 0 on the first tile
            const float pr = actK ? __expf(s[g] - m_new) : 0.f;
            m_run[g] = m_new;
            wv[g] = pr * kvc_scale_value(cur.vsc);
            const float ssum = kvc_warp_sum(pr), zsum = kvc_warp_sum(wv[g] * (float)cur.vmi);
            if (lane == 0) { sm.red[1][warp * G + g] = ssum; sm.red[2][warp * G + g] = zsum; }
        }
        // (the K weights are spent: their memory is the scratch of the V weights' 16-bit values)
        v_weights<G, ROWS>(sm.ps, sm.vstep, sm.red[3], reinterpret_cast<int16_t *>(sm.w), wv, tid);      // three barriers inside
#pragma unroll
        for (int g = 0; g < G; g++) {
            float lt = 0.f;
#pragma unroll
            for (int w8 = 0; w8 < 8; w8++) lt += sm.red[1][w8 * G + g];
            l_run[g] = l_run[g] * alpha[g] + lt;
        }
        const bool v_landed = !BULK || kvc_mbar_wait(&sm.bar[1], par >> 1, p.wait_limit);
        if (BULK && v_landed) par ^= 2u;
        if (!v_landed) flags |= KVC_FLAG_WAIT_TIMEOUT;
        // ---- V: accumulate this tile's contribution for the thread's (group, channel)
        float dv[G];
#pragma unroll
        for (int g = 0; g < G; g++) dv[g] = 0.f;
        if (actV) {
            int hi[G], lo[G];
#pragma unroll
            for (int g = 0; g < G; g++) { hi[g] = 0; lo[g] = 0; }
            bool ok = v_landed && sm.okV[sub] && (uint32_t)(cur.startV >> 3) < sm.nbV[sub];
            if (ok) {
                if constexpr (ROWS) ok = decode_rows<G>(slotsV + sub * p.slotV_bytes, sm.leadV[sub] + (cur.startV >> 3), sm.bookV, escV, myrow, sm.ps + grp * VecWords<G, true>::value, hi, lo);
                else ok = decode_dot<G>(slotsV + sub * p.slotV_bytes, sm.leadV[sub] + (cur.startV >> 3), sm.bookV, escV, sm.ps + grp * VecWords<G, false>::value, hi, lo);
            }
            if (!ok) flags |= KVC_FLAG_BAD_STREAM;
#pragma unroll
            for (int g = 0; g < G; g++)
                dv[g] = fix_value(sm.vstep[grp * G + g], hi[g], lo[g]) +
                        sm.red[2][(grp * 4 + 0) * G + g] + sm.red[2][(grp * 4 + 1) * G + g] +
                        sm.red[2][(grp * 4 + 2) * G + g] + sm.red[2][(grp * 4 + 3) * G + g];
        }
#pragma unroll
        for (int g = 0; g < G; g++) acc[g] = fmaf(acc[g], alpha[g], dv[g]);
        __syncthreads();                                   // every thread is done with the V slots, weights and sums
        if (BULK && warp == 0) {                           // next tile's V blocks land during its K phase
            if (__all_sync(0xffffffffu, v_landed))
                stage_bulk(p.v, validV(n_on, n_tile, lane & 3), blkV_of(n_col, n_tile, lane & 3), slotsV + (lane & 3) * p.slotV_bytes, sm.leadV, sm.okV, sm.nbV, &sm.bar[1], lane, p.starve != 0);
            else if (lane == 0) sm.dead = 1;
        }
        cur = nxt;
    }

    // ---- uncompressed tail (the recent window), handled with the column's last tiles: dense fp16 rows.
    // Only for callers without a workspace: otherwise the merge kernel adds the tail (see there).
    if (p.Tr > 0 && !p.partial && it.t_hi == n_tiles) {
        float *pt = reinterpret_cast<float *>(sm.w);           // p[row][g] for 256 rows
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
    if (it.t_lo >= it.t_hi && have_next) q_fetch(nit.col);     // an item without tiles fetched nothing yet
    const long long head0 = b * Hq + hq0;
    if (!p.partial) {
        // ---- the item is the whole column: combine the CTA's two token groups and write the output
        __syncthreads();
        float *sumbuf = reinterpret_cast<float *>(sm.w);       // [2][128][G]
#pragma unroll
        for (int g = 0; g < G; g++) sumbuf[(grp * 128 + ch) * G + g] = acc[g];
        __syncthreads();
        if (tid < 128) {
#pragma unroll
            for (int g = 0; g < G; g++)
                p.out[(head0 + g) * 128 + tid] = __float2half_rn((sumbuf[tid * G + g] + sumbuf[(128 + tid) * G + g]) / l_run[g]);
        }
    } else {
        // ---- a partial result {m, l, -, -, acc of group 0 [128], acc of group 1 [128]}; a second kernel merges
#pragma unroll
        for (int g = 0; g < G; g++) {
            float *dst = p.ws_part + ((head0 + g) * p.splits + it.part) * ATTN_PART_FLOATS;
            dst[4 + tid] = acc[g];                             // tid = grp * 128 + ch
            if (tid == 0) { dst[0] = m_run[g]; dst[1] = l_run[g]; }
        }
    }
    if (draw && tid == 0) sm.next_j = drawn;
    __syncthreads();                                       // the sums are read before the next column's weights overwrite them
    if (BULK && sm.dead != 0) break;                       // a staging wait ran out: the status word says so, the item's result is void
    const int j_n2 = draw ? 2 * P + sm.next_j : j_n1 + 1;
    it = nit; have = have_next; j_it = j_n1; j_n1 = j_n2;
    have_next = have && item_of(j_n1, nit);
    }   // items of the CTA
    if (BULK && any_tiles) {              // the copies issued after the last tile are empty, but their phase must end;
        // after a wait that ran out, these are the phases still open: nothing may be in flight at the return
        if (!kvc_mbar_wait(&sm.bar[0], par & 1u, p.wait_limit)) flags |= KVC_FLAG_WAIT_TIMEOUT;
        if (!kvc_mbar_wait(&sm.bar[1], par >> 1, p.wait_limit)) flags |= KVC_FLAG_WAIT_TIMEOUT;
    }
    if (flags) atomicOr(p.status, flags);
    if (draw && tid == 0) {               // the last CTA to finish leaves the scheduling counters zeroed for the next launch
        __threadfence();
        if (atomicAdd(&p.sched[1], 1) == (int)gridDim.x - 1) { p.sched[0] = 0; p.sched[1] = 0; __threadfence(); }
    }
}

// The uncompressed tail of a cache (the recent window): dense fp16 rows [Tr, B, Hkv, 128] behind the compressed part.
struct TailArgs {
    const __half *q, *ktail, *vtail;
    long long Tr;
    int B, Hkv, Hq;
    float scaling;
};

// Loads that stay where they are written: a batch of them is issued before the first use (left to itself the
// compiler moves each load down to its use, and the batch becomes a chain of memory round trips).
__device__ __forceinline__ uint4 ld_nc_128_pinned(const void *p) {
    uint4 v;
    asm volatile("ld.global.nc.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
    return v;
}
__device__ __forceinline__ unsigned short ld_nc_16_pinned(const void *p) {
    unsigned short v;
    asm volatile("ld.global.nc.u16 %0, [%1];" : "=h"(v) : "l"(p));
    return v;
}

// Merges the `splits` partial results of every head and adds the tail: grid = heads; 256 threads: the first 128 are the output channels.
//
// The tail is this kernel's work, not the attention kernel's: its rows lie a whole token row apart in memory, so
// every step of it (the query, the K rows, the V rows) is a round trip to memory with little to do in between.
// Inside the attention kernel each column's tail held a 256-thread CTA and its third of an SM for those round
// trips (a 128-row tail lengthened a 137 us launch by 160 us when its loads depended on one another, by 25 us
// with deep batches).  Here every head's tail is in flight at once on small CTAs, and it runs before the
// grid-dependency wait, i.e. while the attention kernel's last CTAs still work: it reads nothing that kernel writes.
// The loads of the partial results are issued in batches before any is used as well.
constexpr int MERGE_THREADS = 256;
__global__ void __launch_bounds__(MERGE_THREADS) attn_merge_kernel(const float *__restrict__ ws_part, __half *__restrict__ out, int splits, TailArgs t) {
    __shared__ float sm_red[8], sm_sum[8], sm_e[128], sm_o[128];
    __shared__ __align__(16) float sm_q[128];
    const float *src = ws_part + (size_t)blockIdx.x * splits * ATTN_PART_FLOATS;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    // launched with programmatic stream serialisation: the kernel behind this one in the stream may set up
    // while this one runs (it touches nothing this one writes before its own wait), and this one's CTAs may be
    // resident before the attention kernel has finished; its partial results are complete and visible after the wait
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    float m_t = -CUDART_INF_F, l_t = 0.f, o_t = 0.f;      // the tail's running maximum and sum; output of channel tid & 127 over the thread's rows
    if (t.Tr > 0) {
        // q.k: two threads per row, 64 channels each; P.V: thread = (half of the pass's rows, channel)
        const int row = tid >> 1, part = tid & 1, ch = tid & 127, rg = tid >> 7;
        const long long b = blockIdx.x / t.Hq, h = (blockIdx.x % t.Hq) / (t.Hq / t.Hkv);
        const long long rstride = (long long)t.B * t.Hkv * 128;                 // halves between two rows of a column
        const __half *kcol = t.ktail + (b * t.Hkv + h) * 128 + part * 64, *vcol = t.vtail + (b * t.Hkv + h) * 128 + ch;
        // Every load of a pass -- the query (first pass), the thread's half row of K, its 64 rows of V -- is issued
        // before the first of them is used: one trip to memory per pass instead of one per step of the softmax.
        const unsigned short qbits = tid < 128 ? ld_nc_16_pinned(t.q + (size_t)blockIdx.x * 128 + tid) : (unsigned short)0;
        for (long long r0 = 0; r0 < t.Tr; r0 += 128) {                        // 128 rows per pass
            const int n_here = (int)min(128ll, t.Tr - r0);
            const bool act = row < n_here;
            uint4 kv[8];
            const __half *kr = kcol + (r0 + min(row, n_here - 1)) * rstride;  // rows beyond the pass: read again, not used
#pragma unroll
            for (int j = 0; j < 8; j++) kv[j] = ld_nc_128_pinned(kr + j * 8);
            unsigned short vv[64];
            const __half *vr = vcol + r0 * rstride;
#pragma unroll
            for (int k = 0; k < 64; k++) vv[k] = ld_nc_16_pinned(vr + min(rg * 64 + k, n_here - 1) * rstride);   // rows beyond the pass: weight 0
            if (r0 == 0 && tid < 128) sm_q[tid] = __half2float(__ushort_as_half(qbits)) * t.scaling;
            __syncthreads();                                                  // sm_q is written; the pass before is done with sm_e
            float sc = -CUDART_INF_F;
            if (act) {
                float a0 = 0.f, a1 = 0.f, a2 = 0.f, a3 = 0.f;                 // four sums: no chain of 64 dependent additions
#pragma unroll
                for (int j = 0; j < 8; j++) {
                    const __half2 *kh = reinterpret_cast<const __half2 *>(&kv[j]);
                    const float4 q0 = *reinterpret_cast<const float4 *>(&sm_q[part * 64 + j * 8]);
                    const float4 q1 = *reinterpret_cast<const float4 *>(&sm_q[part * 64 + j * 8 + 4]);
                    const float2 k0 = __half22float2(kh[0]), k1 = __half22float2(kh[1]), k2 = __half22float2(kh[2]), k3 = __half22float2(kh[3]);
                    a0 = fmaf(k0.x, q0.x, a0); a1 = fmaf(k0.y, q0.y, a1); a2 = fmaf(k1.x, q0.z, a2); a3 = fmaf(k1.y, q0.w, a3);
                    a0 = fmaf(k2.x, q1.x, a0); a1 = fmaf(k2.y, q1.y, a1); a2 = fmaf(k3.x, q1.z, a2); a3 = fmaf(k3.y, q1.w, a3);
                }
                sc = (a0 + a1) + (a2 + a3);
            }
            const float other = __shfl_xor_sync(0xffffffffu, sc, 1);          // the row's other half (both -inf beyond the tail)
            sc = act ? sc + other : sc;
            const float mx = kvc_warp_max(sc);
            if (lane == 0) sm_red[warp] = mx;
            __syncthreads();
            float mt = sm_red[0];
#pragma unroll
            for (int w = 1; w < 8; w++) mt = fmaxf(mt, sm_red[w]);
            const float m_new = fmaxf(m_t, mt);
            const float alpha = __expf(m_t - m_new);                          // exp(-inf) = 0 in the first pass
            const float pr = act ? __expf(sc - m_new) : 0.f;
            if (part == 0) sm_e[row] = pr;
            const float ps = kvc_warp_sum(part == 0 ? pr : 0.f);
            if (lane == 0) sm_sum[warp] = ps;
            __syncthreads();
            float lsum = 0.f;
#pragma unroll
            for (int w = 0; w < 8; w++) lsum += sm_sum[w];
            l_t = l_t * alpha + lsum;
            m_t = m_new;
            float d0 = 0.f, d1 = 0.f, d2 = 0.f, d3 = 0.f;                     // rows rg * 64 .. + 63 of the pass, four sums
#pragma unroll
            for (int k = 0; k < 64; k += 4) {
                d0 = fmaf(sm_e[rg * 64 + k], __half2float(__ushort_as_half(vv[k])), d0);
                d1 = fmaf(sm_e[rg * 64 + k + 1], __half2float(__ushort_as_half(vv[k + 1])), d1);
                d2 = fmaf(sm_e[rg * 64 + k + 2], __half2float(__ushort_as_half(vv[k + 2])), d2);
                d3 = fmaf(sm_e[rg * 64 + k + 3], __half2float(__ushort_as_half(vv[k + 3])), d3);
            }
            o_t = fmaf(o_t, alpha, (d0 + d1) + (d2 + d3));
        }
        __syncthreads();                                                      // sm_red and sm_e serve the merge below
        if (tid >= 128) sm_o[tid - 128] = o_t;                                // the second half of the rows joins the first
        __syncthreads();
        if (tid < 128) o_t += sm_o[tid];
    }
    asm volatile("griddepcontrol.wait;" ::: "memory");
    float M = -CUDART_INF_F;                              // the maximum over all partial results
    for (int s2 = tid; s2 < splits; s2 += MERGE_THREADS) M = fmaxf(M, src[(size_t)s2 * ATTN_PART_FLOATS]);
    M = kvc_warp_max(M);
    if (lane == 0) sm_red[warp] = M;
    __syncthreads();
    M = m_t;
#pragma unroll
    for (int w = 0; w < 8; w++) M = fmaxf(M, sm_red[w]);
    float O = 0.f, L = 0.f;                               // O: channel tid of threads 0..127 (the others idle along)
    const int c = tid & 127;
    for (int s0 = 0; s0 < splits; s0 += 128) {
        const int ns = min(128, splits - s0);
        __syncthreads();                                  // the weights of the batch before are spent
        if (tid < 128) {
            float e = 0.f;
            if (tid < ns) {
                const float *pp = src + (size_t)(s0 + tid) * ATTN_PART_FLOATS;
                const float m2 = pp[0];
                e = m2 == -CUDART_INF_F ? 0.f : __expf(m2 - M);
                L = fmaf(pp[1], e, L);
            }
            sm_e[tid] = e;
        }
        __syncthreads();
        if (tid < 128) {
            for (int i0 = 0; i0 < ns; i0 += 8) {          // channel c of 8 partial results, all loads in flight together
                float a[8];
#pragma unroll
                for (int k = 0; k < 8; k++) {
                    const float *pp = src + (size_t)(s0 + min(i0 + k, ns - 1)) * ATTN_PART_FLOATS;
                    a[k] = pp[4 + c] + pp[4 + 128 + c];
                }
#pragma unroll
                for (int k = 0; k < 8; k++) if (i0 + k < ns) O = fmaf(a[k], sm_e[i0 + k], O);
            }
        }
    }
    L = kvc_warp_sum(L);
    __syncthreads();
    if (lane == 0) sm_red[warp] = L;
    __syncthreads();
    L = 0.f;
#pragma unroll
    for (int w = 0; w < 4; w++) L += sm_red[w];           // warps 0..3 hold the partial results' sums
    const float e_t = m_t == -CUDART_INF_F ? 0.f : __expf(m_t - M);
    O = fmaf(o_t, e_t, O);
    L = fmaf(l_t, e_t, L);
    if (tid < 128) out[(size_t)blockIdx.x * 128 + tid] = __float2half_rn(O / L);
}

// Launch with programmatic stream serialisation: the grid may be set up on the device while the kernel
// ahead of it in the stream still runs.  Such a kernel starts with griddepcontrol.wait, which returns
// when that kernel has completed and its writes are visible.
template <class... KArgs, class... Args>
int launch_overlapped(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream, Args... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid; cfg.blockDim = block; cfg.dynamicSmemBytes = smem; cfg.stream = stream;
    cudaLaunchAttribute attr = {};
    attr.id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr.val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = &attr; cfg.numAttrs = 1;
    KVC_CUDA_OK(cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...));
    return KVC_OK;
}

template <class K>
int set_smem(K kernel, size_t bytes) {
    cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)bytes);
    if (e == cudaSuccess) e = cudaFuncSetAttribute(kernel, cudaFuncAttributePreferredSharedMemoryCarveout, 100);
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
    if (is_k) {
        KVC_REQUIRE(c->q.sc == 0 || c->q.tok_div % 64 == 0,
                    "%s: K units that depend on the channel must cover whole 64-token blocks", who);
        // the kernels fetch the units of 4 neighbouring channels with one load
        KVC_REQUIRE(c->q.sc == 0 || (c->q.sc == 1 && c->q.sj % 4 == 0 && c->q.sb % 4 == 0 && c->q.sh % 4 == 0 &&
                                     (reinterpret_cast<uintptr_t>(c->q.scale) & 7) == 0 &&
                                     (reinterpret_cast<uintptr_t>(c->q.min_int) & (c->q.min_bytes == 1 ? 3 : 7)) == 0),
                    "%s: per-channel K units must be contiguous over the channels and 8-byte aligned", who);
    }
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

// Diagnostics for tests of the bounded waits (kvc_attn_debug): process-wide, read at every launch.
static int g_wait_limit = 0, g_starve = 0;
extern "C" void kvc_attn_debug(int wait_limit, int starve) { g_wait_limit = wait_limit; g_starve = starve; }

// CTAs per SM the attention kernel is launched with at most (its launch bounds ask for this many)
constexpr int ATTN_CTAS_PER_SM = 3;
// items a resident CTA should get on average: enough that the draws even out the CTAs' speeds and the
// last items end close together, few enough that the per-item work (q, partial results) stays small
constexpr int ATTN_ITEMS_PER_CTA = 4;

// How the columns are cut when the caller leaves it to the library: long runs of `tps` tiles, and at the
// end of every column short runs of half that, enough of them that each resident CTA finds about two
// short items to finish with.  The short items are handed out last (the item order puts them behind
// all long ones), so the CTAs of a launch end within one short item of each other.
struct RunPlan { int tps, long_runs, short_tiles, splits; };
static RunPlan plan_runs(long long n_tiles, long long cols, int sm_count) {
    RunPlan r = {1, 1, 1, 1};
    if (n_tiles <= 0 || cols <= 0) { r.tps = 0; r.long_runs = 1; r.short_tiles = 0; return r; }
    const long long P = (long long)ATTN_CTAS_PER_SM * sm_count;
    long long tps = cols * n_tiles / (P * ATTN_ITEMS_PER_CTA);       // tiles per long item
    if (tps < 1) tps = 1;
    if (tps > n_tiles) tps = n_tiles;
    // (items of a single tile pay the per-item work too often: measured slower than no short runs at all)
    long long short_tiles = tps >= 4 ? tps / 2 : tps;
    long long short_region = 0;                                      // tiles of a column cut into short runs
    if (short_tiles < tps) {
        short_region = (2 * P * short_tiles + cols - 1) / cols;       // about two short items per CTA over all columns
        short_region = (short_region + tps - 1) / tps * tps;
        if (short_region > n_tiles) short_region = n_tiles;
    }
    long long long_runs = (n_tiles - short_region) / tps;
    short_region = n_tiles - long_runs * tps;
    const long long short_runs = (short_region + short_tiles - 1) / short_tiles;
    r.tps = (int)tps; r.long_runs = (int)long_runs; r.short_tiles = (int)short_tiles; r.splits = (int)(long_runs + short_runs);
    return r;
}

extern "C" int kvc_attn_splits(int64_t T, int64_t B, int64_t Hkv, int sm_count) {
    if (T <= 0 || B <= 0 || Hkv <= 0) return 1;
    if (sm_count <= 0) sm_count = kvc_sm_count();
    return plan_runs((T + 255) / 256, B * Hkv, sm_count).splits;
}

// bytes of the zero-initialised head of a workspace: the two scheduling counters
constexpr int64_t ATTN_COUNTER_BYTES = 256;

extern "C" int64_t kvc_attn_workspace(int64_t B, int64_t Hq, int splits) {
    if (splits < 1) splits = 1;
    return ATTN_COUNTER_BYTES + B * Hq * (int64_t)(splits > 1 ? splits : 1) * ATTN_PART_FLOATS * 4;    // one run still leaves a partial result when a tail follows
}

extern "C" int kvc_attn_decode(const kvc_cache *k, const kvc_cache *v, int64_t T, int64_t B, int64_t Hkv, int64_t Hq,
                               const void *q, float scaling, const void *ktail, const void *vtail, int64_t Tr,
                               void *out, int splits, void *workspace, int64_t workspace_bytes,
                               int32_t *status, kvc_stream_t stream) {
    if (T > 0) {      // with nothing compressed yet only the fp16 tail is read and the caches may be NULL
        if (int rc = check_cache(k, "kvc_attn_decode", true)) return rc;
        if (int rc = check_cache(v, "kvc_attn_decode", false)) return rc;
    }
    KVC_REQUIRE(q && out && status, "kvc_attn_decode: null pointer");
    KVC_REQUIRE(B > 0 && Hkv > 0 && Hq > 0 && Hq % Hkv == 0, "kvc_attn_decode: bad head counts");
    KVC_REQUIRE(T >= 0 && T % 128 == 0, "kvc_attn_decode: the compressed length must be a multiple of 128, got %lld", (long long)T);
    KVC_REQUIRE(Tr >= 0 && (Tr == 0 || (ktail && vtail)), "kvc_attn_decode: tail pointers missing");
    KVC_REQUIRE(T + Tr > 0, "kvc_attn_decode: empty cache");
    KVC_REQUIRE(Tr == 0 || ((reinterpret_cast<uintptr_t>(ktail) & 15) == 0), "kvc_attn_decode: ktail must be 16-byte aligned");
    const long long n_tiles = (T + 255) / 256, cols = B * Hkv;
    KVC_REQUIRE(T < (1ll << 31) - 1024 && cols < (1ll << 30) && B * Hq < (1ll << 30), "kvc_attn_decode: shape too large");
    // every column is cut into runs of tiles; each (column, run) is one item of work.  splits > 0: that many
    // equal runs.  Otherwise long runs and, at the end of each column, short ones (plan_runs).
    int tps, long_runs, short_tiles;
    if (splits <= 0) {
        const RunPlan r = plan_runs(n_tiles, cols, kvc_sm_count());
        tps = r.tps; long_runs = r.long_runs; short_tiles = r.short_tiles; splits = r.splits;
    } else {
        if (splits > n_tiles) splits = (int)(n_tiles > 0 ? n_tiles : 1);
        tps = (int)((n_tiles + splits - 1) / splits);
        splits = tps > 0 ? (int)((n_tiles + tps - 1) / tps) : 1;
        long_runs = splits; short_tiles = tps;
    }
    KVC_REQUIRE(cols * splits < (1ll << 31) - (1ll << 20), "kvc_attn_decode: too many items");
    if (splits > 1) {
        KVC_REQUIRE(workspace && workspace_bytes >= kvc_attn_workspace(B, Hq, splits),
                    "kvc_attn_decode: workspace needs %lld bytes for %d splits", (long long)kvc_attn_workspace(B, Hq, splits), splits);
        KVC_REQUIRE((reinterpret_cast<uintptr_t>(workspace) & 15) == 0, "kvc_attn_decode: workspace must be 16-byte aligned");
    }
    AttnParams p;
    if (T > 0) { p.k = to_dev(*k); p.v = to_dev(*v); }
    else { p.k = CacheDev(); p.v = CacheDev(); p.k.q.tok_div = p.v.q.tok_div = 1; }
    p.T = T; p.B = B; p.Hkv = Hkv; p.Hq = Hq; p.Tr = Tr;
    p.q = reinterpret_cast<const __half *>(q);
    p.ktail = reinterpret_cast<const __half *>(ktail); p.vtail = reinterpret_cast<const __half *>(vtail);
    p.out = reinterpret_cast<__half *>(out);
    p.scaling = scaling; p.splits = splits; p.tiles_per_split = tps; p.long_runs = long_runs; p.short_tiles = short_tiles;
    p.n_tiles = (int)n_tiles;
    p.work = cols * splits;
    // with a workspace the CTAs draw their items from its counters (zero before the first launch, left zeroed)
    const bool have_ws = workspace && workspace_bytes >= ATTN_COUNTER_BYTES && (reinterpret_cast<uintptr_t>(workspace) & 15) == 0;
    p.sched = have_ws ? reinterpret_cast<int *>(workspace) : nullptr;
    p.ws_part = have_ws ? reinterpret_cast<float *>(reinterpret_cast<uint8_t *>(workspace) + ATTN_COUNTER_BYTES) : nullptr;
    // The tail belongs to the merge kernel whenever the attention kernel can leave partial results for it (a
    // workspace with room for them) or has nothing to do at all (no compressed part); only a caller without a
    // workspace gets the tail from the attention kernel itself.
    const bool ws_parts = have_ws && workspace_bytes >= kvc_attn_workspace(B, Hq, splits);
    const bool tail_in_merge = Tr > 0 && (T == 0 || splits > 1 || ws_parts);
    p.partial = splits > 1 || (tail_in_merge && T > 0);
    p.status = status;
    p.wait_limit = g_wait_limit > 0 ? g_wait_limit : KVC_WAIT_LIMIT;
    p.starve = g_starve;
    // a slot holds the largest block plus its alignment lead, widened to 16-byte chunks, plus the
    // decoder's two words of read-ahead
    p.slotK_bytes = ((p.k.max_block + 15u + 15u) & ~15u) + 16u;
    p.slotV_bytes = ((p.v.max_block + 15u + 15u) & ~15u) + 16u;
    const size_t slot_total = 4 * (size_t)(p.slotK_bytes + p.slotV_bytes) + SLOT_PAD;
    // bulk copies widen every block to 16-byte boundaries: both streams must start on one
    const bool bulk = T > 0 && (reinterpret_cast<uintptr_t>(k->encoded) & 15) == 0 && (reinterpret_cast<uintptr_t>(v->encoded) & 15) == 0;
    const int sms = kvc_sm_count();
    const long long Gt = Hq / Hkv;
    for (long long g0 = 0; g0 < Gt && !(T == 0 && tail_in_merge);) {       // nothing compressed: the merge kernel alone
        const int G = next_chunk(Gt - g0);
        p.g0 = g0;
#define KVC_AT(GG, BB)                                                                                          \
    {                                                                                                           \
        const size_t smem = slot_total + sizeof(AttnSmem<GG>) + ((GG) >= 2 ? NTHR * ROW_STRIDE : 0);               \
        if (int rc = set_smem(attn_decode_kernel<GG, BB>, smem)) return rc;                                     \
        int occ = 0;                                                                                            \
        KVC_CUDA_OK(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&occ, attn_decode_kernel<GG, BB>, NTHR, smem)); \
        KVC_REQUIRE(occ >= 1, "kvc_attn_decode: %zu bytes of shared memory do not fit an SM", smem);             \
        long long ctas = (long long)sms * (occ < ATTN_CTAS_PER_SM ? occ : ATTN_CTAS_PER_SM);                    \
        if (ctas > p.work) ctas = p.work;                                                                       \
        if (int rc = launch_overlapped(attn_decode_kernel<GG, BB>, dim3((unsigned)ctas), dim3(NTHR), smem, kvc_cu(stream), p)) return rc; \
    }
        if (bulk) { if (G == 4) KVC_AT(4, true) else if (G == 2) KVC_AT(2, true) else KVC_AT(1, true) }
        else { if (G == 4) KVC_AT(4, false) else if (G == 2) KVC_AT(2, false) else KVC_AT(1, false) }
#undef KVC_AT
        g0 += G;
    }
    if (p.partial || tail_in_merge) {
        TailArgs ta = {};
        if (tail_in_merge) {
            ta.q = p.q; ta.ktail = p.ktail; ta.vtail = p.vtail; ta.Tr = Tr;
            ta.B = (int)B; ta.Hkv = (int)Hkv; ta.Hq = (int)Hq; ta.scaling = scaling;
        }
        if (int rc = launch_overlapped(attn_merge_kernel, dim3((unsigned)(B * Hq)), dim3(MERGE_THREADS), 0, kvc_cu(stream),
                                       (const float *)p.ws_part, p.out, T > 0 ? splits : 0, ta)) return rc;
    }
    KVC_LAUNCH_OK();
    return KVC_OK;
}

// ---- decode attention for callers that cannot allocate device memory ------------------------------
// Some hosts of this library may not call cudaMalloc at all: an inference server whose memory pool
// owns every byte of the device and forbids side allocations, a plugin loaded into a process that
// runs under a fixed memory budget, or code that runs where an allocation would synchronise the
// device at the wrong moment.  For them the split-KV scratch of the attention kernel (per-head
// counters and the per-split partial results) lives in this fixed array instead of a workspace the
// caller has to provide.  Every GPU that loads the library holds these bytes until the process exits.
#define KVC_STATIC_SCRATCH_BYTES (4 << 20)
static __device__ __align__(256) unsigned char g_attn_scratch[KVC_STATIC_SCRATCH_BYTES];

namespace {
constexpr int MAX_DEVICES = 64;
std::mutex g_scratch_mutex;
void *g_scratch_ptr[MAX_DEVICES] = {};

// The array's name is only a host-side handle in host code; the device address has to be asked for,
// once per device, with that device current.
int static_scratch(void **ptr) {
    int dev = -1;
    KVC_CUDA_OK(cudaGetDevice(&dev));
    KVC_REQUIRE(dev >= 0 && dev < MAX_DEVICES, "kvc_attn_decode_static: device %d out of range", dev);
    std::lock_guard<std::mutex> lock(g_scratch_mutex);
    if (!g_scratch_ptr[dev]) {
        void *p = nullptr;
        KVC_CUDA_OK(cudaGetSymbolAddress(&p, g_attn_scratch));
        g_scratch_ptr[dev] = p;
    }
    *ptr = g_scratch_ptr[dev];
    return KVC_OK;
}
}  // namespace

extern "C" int64_t kvc_attn_static_capacity(void) { return KVC_STATIC_SCRATCH_BYTES; }

extern "C" int kvc_attn_decode_static(const kvc_cache *k, const kvc_cache *v, int64_t T, int64_t B, int64_t Hkv, int64_t Hq,
                                      const void *q, float scaling, const void *ktail, const void *vtail, int64_t Tr,
                                      void *out, int splits, int32_t *status, kvc_stream_t stream) {
    KVC_REQUIRE(B > 0 && Hkv > 0 && Hq > 0 && T >= 0, "kvc_attn_decode_static: bad shape");
    // partial results per head: kvc_attn_decode never cuts a column into more runs than it has tiles
    const long long n_tiles = (T + 255) / 256;
    const int parts = splits <= 0 ? kvc_attn_splits(T, B, Hkv, 0) : (int)(splits > n_tiles ? (n_tiles > 0 ? n_tiles : 1) : splits);
    const int64_t need = kvc_attn_workspace(B, Hq, parts);
    if (need > KVC_STATIC_SCRATCH_BYTES) {
        kvc_set_error("kvc_attn_decode_static: B=%lld x Hq=%lld x %d splits needs %lld bytes of scratch, the built-in "
                      "array holds %d; lower `splits` or use kvc_attn_decode with a workspace",
                      (long long)B, (long long)Hq, parts, (long long)need, KVC_STATIC_SCRATCH_BYTES);
        return KVC_ERR_CAPACITY;
    }
    void *scratch = nullptr;
    if (int rc = static_scratch(&scratch)) return rc;
    // the array keeps whatever the previous call left: the scheduling counters must start at zero
    KVC_CUDA_OK(cudaMemsetAsync(scratch, 0, ATTN_COUNTER_BYTES, kvc_cu(stream)));
    return kvc_attn_decode(k, v, T, B, Hkv, Hq, q, scaling, ktail, vtail, Tr, out, splits, scratch, need, status, stream);
}
