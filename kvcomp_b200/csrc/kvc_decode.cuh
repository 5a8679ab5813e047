// Per-thread Huffman vector decoder shared by the plain decoder and the fused attention kernels.
//
// A vector is 128 symbols, MSB-first, starting on a byte boundary (kernels.cu:237-291 walks it
// one bit at a time through a tree in global memory).  Here the block's bytes sit in shared
// memory, the thread keeps 64 bits of the stream in two registers and looks up KVC_LUT_BITS
// bits at a time in a shared-memory table that returns up to three symbols per lookup; codes
// longer than the window continue bit by bit from the tree node the window leads to.
#pragma once

#include "kvc_common.cuh"

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

// Decode one vector.  sw: the slot as 32-bit words; byte_pos: where the vector starts in the slot.
// emit(s0, s1, s2, ns, c) receives up to three symbols (unused ones are 0) for positions c..c+ns-1;
// it may be handed symbols beyond position 127 at the very end of the vector and must ignore them.
// Every iteration advances by at least one symbol, so the loop ends after at most 128 rounds.
// Word reads are clamped to max_word (the last word of the slot), so a corrupt stream can make the
// result wrong but never the access.  Returns false when the bits do not form valid codes.
template <class Emit>
__device__ __forceinline__ bool kvc_decode_vector(const uint32_t *__restrict__ sw, uint32_t byte_pos,
                                                  uint32_t max_word, const KvcBookSmem &book, Emit emit) {
    uint32_t wi = min(byte_pos >> 2, max_word - 1), p = (byte_pos & 3u) << 3;
    uint32_t hi = kvc_bswap(sw[wi]), lo = kvc_bswap(sw[wi + 1]);
    wi += 2;
    int c = 0;
    bool ok = true;
    while (c < KVC_VEC_LEN) {
        const uint32_t win = __funnelshift_l(lo, hi, p);
        const uint32_t e = book.lut[win >> (32 - KVC_LUT_BITS)];
        const uint32_t ns = (e >> 4) & 3u;
        if (ns != 0) {
            emit((e >> 8) & 0xffu, (e >> 16) & 0xffu, e >> 24, ns, c);
            c += ns;
            p += e & 15u;
        } else {                                       // code longer than the window
            uint32_t node = e >> 8, sym = 0;
            bool found = false;
            p += KVC_LUT_BITS;
            for (int guard = 0; guard < 40; guard++) {
                if (p >= 32) { hi = lo; lo = kvc_bswap(sw[min(wi, max_word)]); wi++; p -= 32; }
                if (node >= 512u) break;
                const uint32_t nd = book.tree[node];
                if ((nd & 0xffffu) == KVC_TREE_LEAF) { sym = nd >> 16; found = true; break; }
                const uint32_t bit = __funnelshift_l(lo, hi, p) >> 31;
                p++;
                node = (nd >> (16 * bit)) & 0xffffu;
            }
            ok = ok && found;
            emit(sym, 0u, 0u, 1u, c);
            c += 1;
        }
        if (p >= 32) { hi = lo; lo = kvc_bswap(sw[min(wi, max_word)]); wi++; p -= 32; }
    }
    return ok;
}
