// Blocked Huffman encoder (kernels.cu:181-235, 419-596 restated for sm_100a).
//
// One launch, one 64-thread CTA per block of 64 vectors, a deterministic stream:
//   sizes   the 64x128 code tile is staged in shared memory once; a thread per vector sums its code
//           lengths, a two-warp scan gives thread_info and the block's byte count
//   encode  the thread shifts its codes through a 64-bit register and ORs whole words into a zeroed
//           shared-memory image of the block (a vector shares its first and last word with its neighbours)
//   offset  the block's place in the stream is the sum of the byte counts of all blocks before it: a chained
//           scan over one state word per block, looked up after the encoding so that the wait is short
//   copy    the image goes out as 128-bit stores, shifted to the destination's alignment on the way
// Books whose symbols are all below 32 (error bounds of 0.05 and more) keep the code table in registers
// and look symbols up with warp shuffles.
#include "kvc_common.cuh"

namespace {

constexpr int TILE_STRIDE = 132;                  // bytes per vector row in shared memory (padded)
constexpr int OUT_CAP = 8192 + 32;                // block image: 8191 bytes max + alignment lead + slack

constexpr int ENC_THREADS = 64;                   // one thread per vector of the block
constexpr int ENC_WAIT_LIMIT = 1 << 21;           // polls of a block's state word (about 40 ns apart) before a CTA gives up

// Stage the code tile of block `blk` as tile[vector][symbol].
// K: vector v = token 64j+v, symbols = its 128 channels (rows of 128 contiguous bytes).
// V: vector v = channel column 64m+v, symbols = tokens 128g..128g+127 (transposed on the way in).
__device__ __forceinline__ void stage_tile(uint8_t *tile, const uint8_t *__restrict__ codes, long long blk,
                                           long long cols, int is_k, int tid) {
    const long long row = cols * 128;
    // K: 16-byte loads, all of a thread's 8 in flight at once (rows are 128 bytes at 16-byte aligned
    // offsets of a 4-byte aligned base: the base decides whether the wide load is legal)
    const bool wide = (reinterpret_cast<uintptr_t>(codes) & 15) == 0;
    if (is_k) {
        const long long j = blk / cols, col = blk % cols;
        const uint8_t *src = codes + (j * 64) * row + col * 128;
        if (wide) {
            uint4 x[8];
#pragma unroll
            for (int k = 0; k < 8; k++) {                       // 64 rows x 8 chunks of 16 bytes
                const int i = tid + k * ENC_THREADS, v = i >> 3, c = i & 7;
                x[k] = *reinterpret_cast<const uint4 *>(src + v * row + c * 16);
            }
#pragma unroll
            for (int k = 0; k < 8; k++) {
                const int i = tid + k * ENC_THREADS, v = i >> 3, c = i & 7;
                uint32_t *d = reinterpret_cast<uint32_t *>(tile + v * TILE_STRIDE + c * 16);
                d[0] = x[k].x; d[1] = x[k].y; d[2] = x[k].z; d[3] = x[k].w;
            }
        } else {
#pragma unroll 8
            for (int i = tid; i < 64 * 32; i += ENC_THREADS) {  // 64 rows x 32 words
                int v = i >> 5, w = i & 31;
                uint32_t x = *reinterpret_cast<const uint32_t *>(src + v * row + w * 4);
                *reinterpret_cast<uint32_t *>(tile + v * TILE_STRIDE + w * 4) = x;
            }
        }
    } else {
        const long long g = blk / (cols * 2), m = blk % (cols * 2);
        const uint8_t *src = codes + (g * 128) * row + m * 64;
        {   // 4-byte loads: 16 lanes cover a token row's 64 bytes, and the transposed stores meet no bank twice
#pragma unroll 2
            for (int i = tid; i < 32 * 16; i += ENC_THREADS) {  // 32 groups of 4 token rows x 16 words of 4 channels
                const int tg = i >> 4, w = i & 15;
                uint32_t x0 = *reinterpret_cast<const uint32_t *>(src + (tg * 4 + 0) * row + w * 4);
                uint32_t x1 = *reinterpret_cast<const uint32_t *>(src + (tg * 4 + 1) * row + w * 4);
                uint32_t x2 = *reinterpret_cast<const uint32_t *>(src + (tg * 4 + 2) * row + w * 4);
                uint32_t x3 = *reinterpret_cast<const uint32_t *>(src + (tg * 4 + 3) * row + w * 4);
                kvc_transpose4x4(x0, x1, x2, x3);               // now one word per channel: its 4 tokens
                *reinterpret_cast<uint32_t *>(tile + (w * 4 + 0) * TILE_STRIDE + tg * 4) = x0;
                *reinterpret_cast<uint32_t *>(tile + (w * 4 + 1) * TILE_STRIDE + tg * 4) = x1;
                *reinterpret_cast<uint32_t *>(tile + (w * 4 + 2) * TILE_STRIDE + tg * 4) = x2;
                *reinterpret_cast<uint32_t *>(tile + (w * 4 + 3) * TILE_STRIDE + tg * 4) = x3;
            }
        }
    }
}

__device__ __forceinline__ uint32_t warp_excl_scan(uint32_t v, int lane, uint32_t *total) {
    uint32_t x = v;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) { uint32_t y = __shfl_up_sync(0xffffffffu, x, o); if (lane >= o) x += y; }
    *total = __shfl_sync(0xffffffffu, x, 31);
    return x - v;
}

// Thread = vector: encode the 128 symbols held in `row` into the block image `out`, starting at byte `start`.
// SHORT: no code is longer than 16 bits.
template <bool SHORT>
__device__ __forceinline__ void encode_vector(const uint32_t (&row)[32], const uint2 *tab, uint32_t *out, uint32_t start) {
    // acc collects code bits below the `have` bits it already holds; whole words leave from the top
    uint32_t wp = start >> 2, have = (start & 3u) * 8;   // the first word's leading bytes belong to the vector before
    unsigned long long acc = 0;
    auto flush = [&]() {
        have -= 32u;
        const uint32_t word = (uint32_t)(acc >> have);
        atomicOr(&out[wp], word);     // only a vector's first and last word can be shared with a neighbour, but one
        wp++;                         // unconditional OR into the zeroed image issues fewer instructions than choosing
    };
#pragma unroll
    for (int w = 0; w < 32; w++) {
        const uint32_t x = row[w];
        const uint2 e0 = tab[x & 0xffu], e1 = tab[(x >> 8) & 0xffu], e2 = tab[(x >> 16) & 0xffu], e3 = tab[x >> 24];
        if (SHORT) {
            // codes of at most 16 bits: two of them make one piece of at most 32 bits, one test per pair
            // (a missing symbol has length 0 and code 0: nothing changes)
            const uint32_t la = e0.y + e1.y, lb = e2.y + e3.y;
            const uint32_t pa = (e0.x << e1.y) | e1.x, pb = (e2.x << e3.y) | e3.x;
            acc = (acc << la) | pa; have += la;
            if (have >= 32u) flush();
            acc = (acc << lb) | pb; have += lb;
            if (have >= 32u) flush();
        } else {
            acc = (acc << e0.y) | e0.x; have += e0.y; if (have >= 32u) flush();
            acc = (acc << e1.y) | e1.x; have += e1.y; if (have >= 32u) flush();
            acc = (acc << e2.y) | e2.x; have += e2.y; if (have >= 32u) flush();
            acc = (acc << e3.y) | e3.x; have += e3.y; if (have >= 32u) flush();
        }
    }
    if (have) atomicOr(&out[wp], (uint32_t)(acc << (32u - have)));   // the tail, zero-padded to a byte by the next start
}

// encode_vector<true> for a book whose symbols are all below 32: the table lives in the warp's registers, lane i
// holding (code << 8) | length of symbol i, and a lookup is a shuffle (one pass of the shared-memory pipe, no
// bank conflicts) instead of a 64-bit shared load at a data-dependent address.  Every lane of the warp must
// call this, with symbols below 32 only (the shuffle reads lane `symbol mod 32`).
__device__ __forceinline__ void encode_vector_shfl(const uint32_t (&row)[32], uint32_t entry, uint32_t *out, uint32_t start) {
    uint32_t wp = start >> 2, have = (start & 3u) * 8;
    unsigned long long acc = 0;
    auto flush = [&]() {
        have -= 32u;
        atomicOr(&out[wp], (uint32_t)(acc >> have));
        wp++;
    };
#pragma unroll
    for (int w = 0; w < 32; w++) {
        const uint32_t x = row[w];
        const uint32_t e0 = __shfl_sync(0xffffffffu, entry, x), e1 = __shfl_sync(0xffffffffu, entry, x >> 8);
        const uint32_t e2 = __shfl_sync(0xffffffffu, entry, x >> 16), e3 = __shfl_sync(0xffffffffu, entry, x >> 24);
        const uint32_t l1 = e1 & 0xffu, l3 = e3 & 0xffu;
        const uint32_t la = (e0 & 0xffu) + l1, lb = (e2 & 0xffu) + l3;
        const uint32_t pa = ((e0 >> 8) << l1) | (e1 >> 8), pb = ((e2 >> 8) << l3) | (e3 >> 8);
        acc = (acc << la) | pa; have += la;
        if (have >= 32u) flush();
        acc = (acc << lb) | pb; have += lb;
        if (have >= 32u) flush();
    }
    if (have) atomicOr(&out[wp], (uint32_t)(acc << (32u - have)));
}

// ---- single pass ------------------------------------------------------------------------------
// One CTA per block does all three phases: the block's byte offset comes from a chained scan over a state
// word per block ({2-bit flag, 62-bit byte count}), so the code tile is read once and no second launch
// waits for the sizes of the first.  A CTA takes its block number from a counter, so every block it
// waits for belongs to a CTA that already runs; each wait is bounded.
constexpr unsigned long long ST_AGG = 1ull << 62;        // value = this block's bytes
constexpr unsigned long long ST_PREFIX = 2ull << 62;     // value = bytes of every block up to and including this one
constexpr unsigned long long ST_DEAD = 3ull << 62;       // a wait ran out at or before this block
constexpr unsigned long long ST_VALUE = ST_AGG - 1;

__device__ __forceinline__ unsigned long long ld_state(const unsigned long long *p) {
    unsigned long long v;
    asm volatile("ld.relaxed.gpu.global.u64 %0, [%1];" : "=l"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ void st_state(unsigned long long *p, unsigned long long v) {
    asm volatile("st.relaxed.gpu.global.u64 [%0], %1;" :: "l"(p), "l"(v) : "memory");
}

// Warp 0: bytes of all blocks before `blk`.  False when a wait ran out (or an earlier block gave up).
// A round trip to memory brings the state of 32 blocks, nearest first; the walk ends at the nearest block
// whose own offset is known.  (Wider rounds of 64 to 256 words measured slower.)
__device__ __forceinline__ bool look_back(const unsigned long long *state, long long blk, int lane, int wait_limit,
                                          unsigned long long *excl_out) {
    unsigned long long mine = 0;                                // this lane's share of the sum
    for (long long idx = blk - 1; idx >= 0; idx -= 32) {
        const long long j = idx - lane;
        unsigned long long v = ST_PREFIX;                       // before the first block: nothing
        int tries = 0;
        for (;;) {
            if (j >= 0) v = ld_state(state + j);
            if (__all_sync(0xffffffffu, (v >> 62) != 0)) break;
            if (++tries > wait_limit) return false;
            __nanosleep(40);
        }
        const unsigned flag = (unsigned)(v >> 62);
        const unsigned dead = __ballot_sync(0xffffffffu, flag == 3u);
        const unsigned pref = __ballot_sync(0xffffffffu, flag == 2u);
        const int first = pref ? __ffs(pref) - 1 : 31;          // the nearest block with a finished prefix
        if (dead & (0xffffffffu >> (31 - first))) return false;
        if (lane <= first) mine += v & ST_VALUE;
        if (pref) break;
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) mine += __shfl_xor_sync(0xffffffffu, mine, o);
    *excl_out = mine;
    return true;
}

__global__ void __launch_bounds__(ENC_THREADS, 16) encode_onepass_kernel(
    const uint8_t *__restrict__ codes, long long cols, int is_k, long long nblk, const uint32_t *__restrict__ enc,
    int n_entries, uint16_t *__restrict__ thread_info, uint2 *__restrict__ block_info, uint32_t base_offset,
    uint8_t *__restrict__ encoded, long long capacity, unsigned int *__restrict__ ticket,
    unsigned long long *__restrict__ state, unsigned long long *__restrict__ total_bytes,
    int *__restrict__ status, int wait_limit, int starve) {
    // the code tile, and after every thread has taken its row into registers, the block image
    __shared__ __align__(16) uint8_t tile[64 * TILE_STRIDE > OUT_CAP ? 64 * TILE_STRIDE : OUT_CAP];
    uint32_t *const out = reinterpret_cast<uint32_t *>(tile);
    __shared__ uint2 tab[256];                              // {code, length}
    __shared__ uint16_t lens[256];                          // length, or 1 << 14 for a symbol without a code
    __shared__ uint32_t wsum[2];
    __shared__ unsigned int s_blk;
    __shared__ unsigned long long s_excl;
    __shared__ int s_dead;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    if (tid == 0) { s_blk = atomicAdd(ticket, 1u); s_dead = 0; }
    int kind = 0;                                           // 1: a code longer than 16 bits, 2: a coded symbol >= 32
    for (int i = tid; i < 256; i += ENC_THREADS) {
        const uint2 e = i < n_entries ? make_uint2(enc[2 * i], enc[2 * i + 1]) : make_uint2(0u, 0u);
        tab[i] = e;
        kind |= (e.y > 16u ? 1 : 0) | (e.y && i >= 32 ? 2 : 0);
        const uint32_t l = min(e.y, 32u);
        lens[i] = (uint16_t)(l ? l : (1u << 14));
    }
    kind = __syncthreads_or(kind);
    const bool long_codes = (kind & 1) != 0;
    const bool small_book = kind == 0;                      // the table fits a warp's registers
    const long long blk = s_blk;
    // lane i: symbol i's (code << 8) | length for the encoding, and its length (or the marker) for the sizes
    const uint32_t my_entry = (tab[lane].x << 8) | tab[lane].y, my_len = lens[lane];
    stage_tile(tile, codes, blk, cols, is_k, tid);
    __syncthreads();
    int flags = 0;
    uint32_t bits = 0;
    const uint32_t *rowp = reinterpret_cast<const uint32_t *>(tile + tid * TILE_STRIDE);
    uint32_t row[32];
#pragma unroll
    for (int w = 0; w < 32; w++) row[w] = rowp[w];
    uint32_t seen = 0;
#pragma unroll
    for (int w = 0; w < 32; w++) seen |= row[w];
    // a symbol >= 32 in the data of a small book has no code; the warp then takes the general path, which drops it
    const bool by_shfl = small_book && !__any_sync(0xffffffffu, (seen & 0xe0e0e0e0u) != 0);
    if (by_shfl) {
#pragma unroll
        for (int w = 0; w < 32; w++) {
            const uint32_t x = row[w];
            bits += __shfl_sync(0xffffffffu, my_len, x) + __shfl_sync(0xffffffffu, my_len, x >> 8) +
                    __shfl_sync(0xffffffffu, my_len, x >> 16) + __shfl_sync(0xffffffffu, my_len, x >> 24);
        }
    } else {
#pragma unroll 8
        for (int w = 0; w < 32; w++) {
            const uint32_t x = rowp[w];
            bits += lens[x & 0xffu] + lens[(x >> 8) & 0xffu] + lens[(x >> 16) & 0xffu] + lens[x >> 24];
        }
    }
    if (bits >> 14) flags |= KVC_FLAG_SYMBOL_MISSING;
    bits &= (1u << 14) - 1;
    const uint32_t n = (bits + 7) >> 3;                      // the vector's bytes
    if (n > (is_k ? 128u : 256u)) flags |= KVC_FLAG_VECTOR_LONG;
    uint32_t wtotal;
    uint32_t start = warp_excl_scan(n, lane, &wtotal);
    if (lane == 31) wsum[warp] = wtotal;
    __syncthreads();                                         // every row is in registers: the tile's memory is free
    if (warp == 1) start += wsum[0];
    const uint32_t nbytes = wsum[0] + wsum[1];
    // kernels.cu:462-465: (end byte << 3) + pad bits
    thread_info[blk * 64 + tid] = (uint16_t)(((start + n) << 3) + (n * 8 - bits));
    const bool fits = nbytes <= 8191u;                       // else its u16 fields cannot describe the block
    // Later blocks may add this block's bytes to their offsets from here on; its own offset is looked up
    // after the encoding, when the blocks before it have long announced theirs.
    if (tid == 0 && !(starve && blk == 0)) st_state(state + blk, (blk > 0 ? ST_AGG : ST_PREFIX) | nbytes);   // the first block's offset is 0
    if (fits) {
        // The image starts at byte 0 of the shared array, whatever the destination's alignment; it is zeroed
        // past the words the copy-out may touch.
        for (uint32_t i = tid; i * 16 < nbytes + 24; i += ENC_THREADS) reinterpret_cast<uint4 *>(out)[i] = make_uint4(0u, 0u, 0u, 0u);
        __syncthreads();
        if (by_shfl) encode_vector_shfl(row, my_entry, out, start);
        else if (long_codes) encode_vector<false>(row, tab, out, start);
        else encode_vector<true>(row, tab, out, start);
    }
    if (warp == 0) {
        unsigned long long excl = 0;
        bool ok = true;
        if (blk > 0) ok = look_back(state, blk, lane, wait_limit, &excl);
        if (lane == 0) {
            if (!(starve && blk == 0)) st_state(state + blk, ok ? (ST_PREFIX | (excl + nbytes)) : ST_DEAD);
            s_excl = excl;
            if (!ok) { s_dead = 1; flags |= KVC_FLAG_WAIT_TIMEOUT; }
        }
    }
    __syncthreads();                                         // the image is complete and the offset known
    if (s_dead) { if (flags) atomicOr(status, flags); return; }
    const long long off = (long long)s_excl;
    const bool room = off + nbytes <= capacity && off + nbytes + base_offset <= 0xffffffffll;     // u32 offsets
    if (tid == 0) {
        block_info[blk] = make_uint2((uint32_t)(off + base_offset), nbytes & 0xffffu);            // {u32, u16, 2 B zero}
        if (!fits) flags |= KVC_FLAG_BLOCK_LONG;
        if (!room) flags |= KVC_FLAG_STREAM_FULL;
        if (total_bytes) {
            atomicMax(total_bytes + 1, (unsigned long long)nbytes);
            if (blk == nblk - 1) total_bytes[0] = (unsigned long long)off + nbytes;
        }
    }
    if (flags) atomicOr(status, flags);
    if (!fits || !room) return;                              // nothing of this block is written
    // Copy-out in 16-byte pieces of the destination.  Image words hold stream bytes most-significant first;
    // destination byte b (counted from the 16-byte boundary at or before the block's first byte) is image
    // byte b - lead, so a destination word is cut from two image words and swapped to memory order.
    uint8_t *dst = encoded + off;
    const uint32_t lead = (uint32_t)(reinterpret_cast<uintptr_t>(dst) & 15);
    const uint32_t end = lead + nbytes;
    const uint32_t sh = ((4u - (lead & 3u)) & 3u) * 8u;
    uint8_t *g0 = dst - lead;                                   // 16-byte aligned
    for (uint32_t ch = tid; ch * 16 < end; ch += ENC_THREADS) {
        const uint32_t b0 = ch * 16, b1 = b0 + 16;
        const int wi = ((int)b0 - (int)lead) >> 2;              // floor: negative only in the first piece
        uint32_t w[5];
#pragma unroll
        for (int k = 0; k < 5; k++) w[k] = wi + k >= 0 ? out[wi + k] : 0u;
        uint4 wv;
        wv.x = kvc_bswap(__funnelshift_l(w[1], w[0], sh)); wv.y = kvc_bswap(__funnelshift_l(w[2], w[1], sh));
        wv.z = kvc_bswap(__funnelshift_l(w[3], w[2], sh)); wv.w = kvc_bswap(__funnelshift_l(w[4], w[3], sh));
        if (b0 >= lead && b1 <= end) {
            *reinterpret_cast<uint4 *>(g0 + b0) = wv;
        } else {                                                // shared with a neighbouring block
            const uint8_t *bytes = reinterpret_cast<const uint8_t *>(&wv);
            for (uint32_t b = (b0 < lead ? lead : b0); b < (b1 < end ? b1 : end); b++) g0[b] = bytes[b - b0];
        }
    }
}

int g_enc_wait_limit = 0, g_enc_starve = 0;

}  // namespace


extern "C" void kvc_encode_debug(int wait_limit, int starve) {
    g_enc_wait_limit = wait_limit > 0 ? wait_limit : 0;
    g_enc_starve = starve != 0;
}

extern "C" int64_t kvc_encode_workspace(int64_t T, int64_t cols, int is_k) {
    int64_t nblk = is_k ? (T / 64) * cols : (T / 128) * cols * 2;
    return 16 + nblk * 8;                                  // the block counter, then a state word per block
}

extern "C" int kvc_encode(const uint8_t *codes, int64_t T, int64_t cols, int is_k,
                          const void *enc_table, int n_entries, uint32_t base_offset,
                          void *block_info, uint16_t *thread_info, uint8_t *encoded, int64_t encoded_capacity,
                          unsigned long long *total_bytes, void *workspace, int64_t workspace_bytes,
                          int32_t *status, kvc_stream_t stream) {
    KVC_REQUIRE(codes && enc_table && block_info && thread_info && encoded && status, "kvc_encode: null pointer");
    KVC_REQUIRE(cols > 0 && T >= 0, "kvc_encode: bad shape");
    KVC_REQUIRE(n_entries >= 1 && n_entries <= 256, "kvc_encode: the encode table has 1..256 entries");
    KVC_REQUIRE(T % (is_k ? 64 : 128) == 0, "kvc_encode: %s needs a multiple of %d tokens, got %lld",
                is_k ? "K" : "V", is_k ? 64 : 128, (long long)T);
    KVC_REQUIRE((reinterpret_cast<uintptr_t>(codes) & 3) == 0 && (reinterpret_cast<uintptr_t>(block_info) & 7) == 0,
                "kvc_encode: codes must be 4-byte and block_info 8-byte aligned");
    cudaStream_t s = kvc_cu(stream);
    const long long nblk = is_k ? (T / 64) * cols : (T / 128) * cols * 2;
    if (total_bytes) KVC_CUDA_OK(cudaMemsetAsync(total_bytes, 0, 8, s));
    if (nblk == 0) return KVC_OK;
    KVC_REQUIRE(nblk < (1ll << 31), "kvc_encode: too many blocks in one call");
    KVC_REQUIRE(workspace && workspace_bytes >= kvc_encode_workspace(T, cols, is_k),
                "kvc_encode: workspace needs %lld bytes", (long long)kvc_encode_workspace(T, cols, is_k));
    KVC_REQUIRE((reinterpret_cast<uintptr_t>(workspace) & 15) == 0, "kvc_encode: workspace must be 16-byte aligned");
    const uint32_t *enc = reinterpret_cast<const uint32_t *>(enc_table);
    KVC_CUDA_OK(cudaMemsetAsync(workspace, 0, 16 + nblk * 8, s));
    encode_onepass_kernel<<<(unsigned)nblk, ENC_THREADS, 0, s>>>(
        codes, cols, is_k, nblk, enc, n_entries, thread_info, reinterpret_cast<uint2 *>(block_info), base_offset, encoded,
        encoded_capacity, reinterpret_cast<unsigned int *>(workspace),
        reinterpret_cast<unsigned long long *>(reinterpret_cast<uint8_t *>(workspace) + 16), total_bytes, status,
        g_enc_wait_limit ? g_enc_wait_limit : ENC_WAIT_LIMIT, g_enc_starve);
    KVC_LAUNCH_OK();
    return KVC_OK;
}
