// Per-thread Huffman vector decoder shared by the plain decoder and the fused attention kernels,
// and the helpers that stage compressed blocks in shared memory.
//
// A vector is 128 symbols, MSB-first, starting on a byte boundary (kernels.cu:237-291 walks it
// one bit at a time through a tree in global memory).  Here the block's bytes sit in shared
// memory, the thread keeps 64 bits of the stream in two registers and looks up KVC_LUT_BITS
// bits at a time in a shared-memory table that returns up to three symbols per lookup; codes
// longer than the window continue bit by bit from the tree node the window leads to.
#pragma once

#include "kvc_common.cuh"

#define KVC_DECODE_UNROLL 1
#define KVC_DECODE_OVERRUN (3 * KVC_DECODE_UNROLL)   // positions past 127 a decoder may emit
#define KVC_DECODE_OVERRUN_PAIR 6                    // ... with two lookups per round (PAIR)

struct KvcBookSmem {                      // per-CTA copy of the decode structures of one book
    uint32_t tree[512];
    uint32_t lut[KVC_LUT_SIZE];
};

__device__ __forceinline__ void kvc_load_book(KvcBookSmem &b, const void *book, int tid, int nthr) {
    const uint4 *src = reinterpret_cast<const uint4 *>(reinterpret_cast<const uint8_t *>(book) + KVC_BOOK_OFF_TREE);
    uint4 *dst = reinterpret_cast<uint4 *>(&b);
    constexpr int N16 = (int)(sizeof(KvcBookSmem) / 16);
    for (int i = tid; i < N16; i += nthr) dst[i] = src[i];
}

// Copy the bytes [off, off+n) of `encoded` into `slot` so that slot and source agree modulo 16:
// the first stream byte lands at slot[lead], lead = address & 15.  Whole 16-byte chunks inside the
// buffer move as 128-bit loads; the ragged edges move bytewise, never touching memory outside
// [encoded, encoded + encoded_bytes).  Returns lead.  All `nthr` threads of the group take part.
__device__ __forceinline__ uint32_t kvc_stage_block(uint8_t *slot, const uint8_t *__restrict__ encoded,
                                                    long long encoded_bytes, long long off, uint32_t n,
                                                    int tid, int nthr) {
    const uint8_t *src = encoded + off;
    const uint32_t lead = (uint32_t)(reinterpret_cast<uintptr_t>(src) & 15);
    const uint8_t *a0 = src - lead;                                  // 16-byte aligned
    const uint32_t chunks = (lead + n + 15) >> 4;
    const uint8_t *lo = encoded, *hi = encoded + encoded_bytes;
    for (uint32_t c = tid; c < chunks; c += nthr) {
        const uint8_t *p = a0 + 16 * c;
        if (p >= lo && p + 16 <= hi) {
            *reinterpret_cast<uint4 *>(slot + 16 * c) = *reinterpret_cast<const uint4 *>(p);
        } else {
            for (int k = 0; k < 16; k++) slot[16 * c + k] = (p + k >= lo && p + k < hi) ? p[k] : (uint8_t)0;
        }
    }
    return lead;
}

// ---- bulk asynchronous copies (TMA, untiled) completing on a shared-memory mbarrier -------------
__device__ __forceinline__ uint32_t kvc_smem_addr(const void *p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void kvc_mbar_init(uint64_t *bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(kvc_smem_addr(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ void kvc_mbar_fence_init() {
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void kvc_mbar_expect_tx(uint64_t *bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(kvc_smem_addr(bar)), "r"(bytes) : "memory");
}
// src and dst 16-byte aligned, bytes a multiple of 16 and > 0
__device__ __forceinline__ void kvc_bulk_g2s(void *dst, const void *src, uint32_t bytes, uint64_t *bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                 ::"r"(kvc_smem_addr(dst)), "l"(src), "r"(bytes), "r"(kvc_smem_addr(bar)) : "memory");
}
// Bounded wait for the phase with the given parity: at most `limit` tries.  Returns false if the phase
// never completed.
#define KVC_WAIT_LIMIT (1 << 22)
__device__ __forceinline__ bool kvc_mbar_wait(uint64_t *bar, uint32_t parity, int limit = KVC_WAIT_LIMIT) {
    const uint32_t a = kvc_smem_addr(bar);
    for (int it = 0; it < limit; it++) {
        uint32_t done;
        asm volatile("{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}"
                     : "=r"(done) : "r"(a), "r"(parity) : "memory");
        if (done) return true;
    }
    return false;
}

__device__ __forceinline__ int kvc_dp4a_us(uint32_t a_u8x4, uint32_t b_s8x4, int c) {
    int d;
    asm("dp4a.u32.s32 %0, %1, %2, %3;" : "=r"(d) : "r"(a_u8x4), "r"(b_s8x4), "r"(c));
    return d;
}
__device__ __forceinline__ int kvc_dp4a_uu(uint32_t a_u8x4, uint32_t b_u8x4, int c) {
    int d;
    asm("dp4a.u32.u32 %0, %1, %2, %3;" : "=r"(d) : "r"(a_u8x4), "r"(b_u8x4), "r"(c));
    return d;
}

__device__ __forceinline__ uint32_t kvc_lds32(uint32_t addr) {
    uint32_t v;
    asm volatile("ld.shared.u32 %0, [%1];" : "=r"(v) : "r"(addr));
    return v;
}
__device__ __forceinline__ uint2 kvc_lds64(uint32_t addr) {
    uint2 v;
    asm volatile("ld.shared.v2.u32 {%0, %1}, [%2];" : "=r"(v.x), "=r"(v.y) : "r"(addr));
    return v;
}

// Whether the decoder has to test every table entry for "no code ends in this window": books with a
// code longer than the window, and books whose code is not complete (a single symbol, or a tree taken
// from a caller's tensor with a missing branch): a corrupt stream can then show bit patterns that
// belong to no code, and the escape-free loop would not advance on them.
__device__ __forceinline__ bool kvc_book_needs_escape(const void *book) {
    return reinterpret_cast<const kvc_book_header *>(book)->escape != 0;    // set for a code beyond the window too
}

// Decode one vector.  slot_s: shared-space address of the staged block (16-byte aligned); byte_pos:
// where the vector starts in it; lut_s / tree_s: shared-space addresses of the book's tables.
// The decoder state is (position << 6) | bit offset into the (hi, lo) register pair, so applying a
// table entry is one add of its low byte.
// emit(e, a): `e` holds up to three symbols in bytes 1..3 for positions c..c+2 of the vector (unused
// bytes are 0; byte 0 is the table entry's advance byte: its bits 6-7 count the symbols); a = (base + c) << SHIFT:
// the position counter starts at `base`, so a consumer that keeps one record of 2^SHIFT bytes per
// position at shared address A passes base = A >> SHIFT and gets the record's address with no add.
// The end of the vector is tested once per KVC_DECODE_UNROLL lookups, so emit may be handed symbols for
// positions up to 127 + KVC_DECODE_OVERRUN; the consumer keeps room for them (zero weights, padding).
// ESC = false is for books whose longest code fits the table window: no escape test in the loop;
// PAIR (with ESC = false only) takes two lookups per round.
// Every round advances by at least one symbol, so the loop ends after at most 128 rounds; a corrupt
// stream can read at most a few hundred bytes past its vector, for which the kernels keep padding
// behind the last slot.  Returns false when the bits do not form valid codes.
template <bool ESC, int SHIFT, class Emit, bool PAIR = false>
__device__ __forceinline__ bool kvc_decode_vector(uint32_t slot_s, uint32_t byte_pos, uint32_t lut_s, uint32_t tree_s,
                                                  uint32_t base, Emit emit) {
    static_assert(SHIFT >= 0 && SHIFT <= 6, "record size");
    constexpr uint32_t AMASK = 0xffffffffu << SHIFT;       // drops the bit-offset bits left below the position
    const uint32_t end = (base + KVC_VEC_LEN) << 6;
    uint32_t ptr = slot_s + (byte_pos & ~3u);
    uint32_t state = (base << 6) | ((byte_pos & 3u) << 3);
    uint32_t hi = kvc_bswap(kvc_lds32(ptr)), lo = kvc_bswap(kvc_lds32(ptr + 4));
    if (PAIR && !ESC) {
        // Two lookups per round.  The first leaves the bit offset below 32 + KVC_LUT_BITS, so the second
        // one's window still lies inside (hi, lo) or (lo, next word) and needs no refill in between:
        // one refill test and one end test per pair.  The second lookup may run although the first
        // finished the vector, so up to KVC_DECODE_OVERRUN_PAIR positions past 127 are emitted.
        uint32_t nx = kvc_bswap(kvc_lds32(ptr + 8));
        ptr += 12;
        do {
            const uint32_t w0 = __funnelshift_l(lo, hi, state);
            const uint32_t e0 = kvc_lds32(lut_s + ((w0 >> (32 - KVC_LUT_BITS - 2)) & ((KVC_LUT_SIZE - 1) << 2)));
            emit(e0, (state >> (6 - SHIFT)) & AMASK);
            state = (uint32_t)kvc_dp4a_uu(e0, 1u, (int)state);
            const bool up = (state & 32u) != 0;
            const uint32_t w1 = __funnelshift_l(up ? nx : lo, up ? lo : hi, state);
            const uint32_t e1 = kvc_lds32(lut_s + ((w1 >> (32 - KVC_LUT_BITS - 2)) & ((KVC_LUT_SIZE - 1) << 2)));
            emit(e1, (state >> (6 - SHIFT)) & AMASK);
            state = (uint32_t)kvc_dp4a_uu(e1, 1u, (int)state);
            if (state & 32u) { hi = lo; lo = nx; nx = kvc_bswap(kvc_lds32(ptr)); ptr += 4; state -= 32u; }
        } while (state < end);
        return true;
    }
    uint32_t nxt = kvc_lds32(ptr + 8);     // one word of read-ahead keeps the refill off the critical path
    ptr += 12;
    bool ok = true;
    do {
#pragma unroll
      for (int rep = 0; rep < KVC_DECODE_UNROLL; rep++) {             // the end test runs once per UNROLL lookups
        const uint32_t win = __funnelshift_l(lo, hi, state);          // the shift uses the low 5 bits
        const uint32_t e = kvc_lds32(lut_s + ((win >> (32 - KVC_LUT_BITS - 2)) & ((KVC_LUT_SIZE - 1) << 2)));
        if (!ESC || (e & 0xffu) != 0) {
            emit(e, (state >> (6 - SHIFT)) & AMASK);
            state = (uint32_t)kvc_dp4a_uu(e, 1u, (int)state);         // state += byte 0 of e, off the integer ALU pipe
        } else {                                                      // code longer than the window
            uint32_t node = e >> 8, sym = 0;
            bool found = false;
            const uint32_t a = (state >> (6 - SHIFT)) & AMASK;
            state += KVC_LUT_BITS;
            for (int guard = 0; guard < 40; guard++) {
                if (state & 32u) { hi = lo; lo = kvc_bswap(nxt); nxt = kvc_lds32(ptr); ptr += 4; state -= 32u; }
                if (node >= 512u) break;
                const uint32_t nd = kvc_lds32(tree_s + node * 4);
                if ((nd & 0xffffu) == KVC_TREE_LEAF) { sym = nd >> 16; found = true; break; }
                const uint32_t bit = __funnelshift_l(lo, hi, state) >> 31;
                state += 1u;
                node = (nd >> (16 * bit)) & 0xffffu;
            }
            ok = ok && found;
            emit((sym << 8) | (1u << 6), a);                          // advance byte: one symbol
            state += 1u << 6;
        }
        if (state & 32u) { hi = lo; lo = kvc_bswap(nxt); nxt = kvc_lds32(ptr); ptr += 4; state -= 32u; }
      }
    } while (state < end);
    return ok;
}
