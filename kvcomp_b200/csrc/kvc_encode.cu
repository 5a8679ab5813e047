// Blocked Huffman encoder (kernels.cu:181-235, 419-596 restated for sm_100a).
//
// Three phases, no inter-CTA waiting and a deterministic stream:
//   A  sizes   one 64-thread CTA per block: stage the 64x128 code tile in shared memory, a thread
//              per vector sums its code lengths, a two-warp scan -> thread_info, block byte count
//   B  scan    exclusive prefix sum of block byte counts -> block_info offsets (ascending id)
//   C  emit    one 64-thread CTA per block: a thread per vector shifts its codes through a 64-bit
//              register and ORs whole words into a zeroed shared-memory image of the block that is
//              aligned like its destination (a vector shares its first and last word with its
//              neighbours); the image goes out as 128-bit stores
#include "kvc_common.cuh"

namespace {

constexpr int TILE_STRIDE = 132;                  // bytes per vector row in shared memory (padded)
constexpr int OUT_CAP = 8192 + 32;                // block image: 8191 bytes max + alignment lead + slack

constexpr int ENC_THREADS = 64;                   // one thread per vector of the block

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

// ---- phase A ----------------------------------------------------------------------------------
__global__ void __launch_bounds__(ENC_THREADS) encode_sizes_kernel(
    const uint8_t *__restrict__ codes, long long cols, int is_k, const uint32_t *__restrict__ enc, int n_entries,
    uint16_t *__restrict__ thread_info, uint32_t *__restrict__ sizes, unsigned long long *__restrict__ partial,
    unsigned long long *__restrict__ max_block, int *__restrict__ status) {
    __shared__ __align__(16) uint8_t tile[64 * TILE_STRIDE];
    // code lengths as 16-bit entries; a symbol without a code counts 1 << 14 instead, so that the sum of a
    // vector (at most 128 * 32 bits) tells both its length and whether a symbol was missing, with no
    // test per symbol
    __shared__ uint16_t lens[256];
    __shared__ uint32_t wsum[2];
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const long long blk = blockIdx.x;
    for (int i = tid; i < 256; i += ENC_THREADS) {
        const uint32_t l = i < n_entries ? min(enc[2 * i + 1], 32u) : 0u;
        lens[i] = (uint16_t)(l ? l : (1u << 14));
    }
    stage_tile(tile, codes, blk, cols, is_k, tid);
    __syncthreads();
    int flags = 0;
    uint32_t bits = 0;
    const uint32_t *rowp = reinterpret_cast<const uint32_t *>(tile + tid * TILE_STRIDE);
#pragma unroll 8
    for (int w = 0; w < 32; w++) {
        const uint32_t x = rowp[w];
#pragma unroll
        for (int k = 0; k < 4; k++) bits += lens[(x >> (8 * k)) & 0xffu];
    }
    if (bits >> 14) flags |= KVC_FLAG_SYMBOL_MISSING;
    bits &= (1u << 14) - 1;
    const uint32_t n = (bits + 7) >> 3;                      // the vector's bytes
    if (n > (is_k ? 128u : 256u)) flags |= KVC_FLAG_VECTOR_LONG;
    uint32_t wtotal;
    uint32_t start = warp_excl_scan(n, lane, &wtotal);
    if (lane == 31) wsum[warp] = wtotal;
    __syncthreads();
    if (warp == 1) start += wsum[0];
    const uint32_t end = start + n;
    // kernels.cu:462-465: (end byte << 3) + pad bits
    thread_info[blk * 64 + tid] = (uint16_t)((end << 3) + (n * 8 - bits));
    if (tid == 63) {
        const uint32_t total = end;
        sizes[blk] = total;
        atomicAdd(&partial[blk >> 10], (unsigned long long)total);
        if (max_block) atomicMax(max_block, (unsigned long long)total);
        if (total > 8191u) flags |= KVC_FLAG_BLOCK_LONG;
    }
    if (flags) atomicOr(status, flags);
}

// ---- phase B ----------------------------------------------------------------------------------
// partial[i] = byte count of blocks [1024 i, 1024 i + 1024); turn it into an exclusive prefix and
// leave the grand total in partial[n_part].
__global__ void __launch_bounds__(1024) scan_partials_kernel(unsigned long long *__restrict__ partial, long long n_part,
                                                             unsigned long long *__restrict__ total_out) {
    __shared__ unsigned long long wsum[32];
    __shared__ unsigned long long carry;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    if (tid == 0) carry = 0;
    __syncthreads();
    for (long long base = 0; base < n_part; base += 1024) {
        long long i = base + tid;
        unsigned long long v = i < n_part ? partial[i] : 0ull, x = v;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) { unsigned long long y = __shfl_up_sync(0xffffffffu, x, o); if (lane >= o) x += y; }
        if (lane == 31) wsum[warp] = x;
        __syncthreads();
        if (warp == 0) {
            unsigned long long w = wsum[lane], z = w;
#pragma unroll
            for (int o = 1; o < 32; o <<= 1) { unsigned long long y = __shfl_up_sync(0xffffffffu, z, o); if (lane >= o) z += y; }
            wsum[lane] = z - w;
        }
        __syncthreads();
        unsigned long long excl = carry + wsum[warp] + x - v;
        if (i < n_part) partial[i] = excl;
        __syncthreads();
        if (tid == 1023) carry = excl + v;
        __syncthreads();
    }
    if (tid == 0) { partial[n_part] = carry; if (total_out) *total_out = carry; }
}

__global__ void __launch_bounds__(1024) scan_blocks_kernel(const uint32_t *__restrict__ sizes, long long nblk,
                                                           const unsigned long long *__restrict__ partial,
                                                           uint32_t base_offset, long long capacity,
                                                           uint2 *__restrict__ block_info, int *__restrict__ status) {
    __shared__ uint32_t wsum[32];
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const long long i = (long long)blockIdx.x * 1024 + tid;
    uint32_t v = i < nblk ? sizes[i] : 0u, total;
    uint32_t x = warp_excl_scan(v, lane, &total);
    if (lane == 31) wsum[warp] = total;
    __syncthreads();
    if (warp == 0) { uint32_t w = wsum[lane], t2; uint32_t z = warp_excl_scan(w, lane, &t2); wsum[lane] = z; }
    __syncthreads();
    if (i < nblk) {
        unsigned long long off = partial[blockIdx.x] + wsum[warp] + x;
        int flags = 0;
        if ((long long)(off + v) > capacity) flags |= KVC_FLAG_STREAM_FULL;
        if (off + v + base_offset > 0xffffffffull) flags |= KVC_FLAG_STREAM_FULL;     // u32 offsets
        block_info[i] = make_uint2((uint32_t)(off + base_offset), v & 0xffffu);      // {u32, u16, 2 B zero}
        if (flags) atomicOr(status, flags);
    }
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

// ---- phase C ----------------------------------------------------------------------------------
__global__ void __launch_bounds__(ENC_THREADS) encode_emit_kernel(
    const uint8_t *__restrict__ codes, long long cols, int is_k, const uint32_t *__restrict__ enc, int n_entries,
    const uint16_t *__restrict__ thread_info, const uint2 *__restrict__ block_info,
    const uint32_t *__restrict__ sizes, uint32_t base_offset, uint8_t *__restrict__ encoded, long long capacity) {
    // the code tile, and after every thread has taken its row into registers, the block image
    __shared__ __align__(16) uint8_t tile[64 * TILE_STRIDE > OUT_CAP ? 64 * TILE_STRIDE : OUT_CAP];
    uint32_t *const out = reinterpret_cast<uint32_t *>(tile);
    __shared__ uint2 tab[256];                              // {code, length}
    __shared__ uint16_t tinfo[64];
    const int tid = threadIdx.x;
    const long long blk = blockIdx.x;
    const uint2 bi = block_info[blk];
    const long long off = (long long)bi.x - base_offset;
    const uint32_t nbytes = sizes[blk];
    // an oversized block cannot be described by its u16 fields; a full stream has no room: skip
    if (nbytes > 8191u || off + nbytes > capacity) return;
    int too_long = 0;
    for (int i = tid; i < 256; i += ENC_THREADS) {
        tab[i] = i < n_entries ? make_uint2(enc[2 * i], enc[2 * i + 1]) : make_uint2(0u, 0u);
        too_long |= tab[i].y > 16u;
    }
    stage_tile(tile, codes, blk, cols, is_k, tid);
    tinfo[tid] = thread_info[blk * 64 + tid];
    uint8_t *dst = encoded + off;
    const uint32_t lead = (uint32_t)(reinterpret_cast<uintptr_t>(dst) & 15);   // image is aligned like dst
    const uint32_t end = lead + nbytes;
    const bool long_codes = __syncthreads_or(too_long) != 0;
    uint32_t row[32];
#pragma unroll
    for (int w = 0; w < 32; w++) row[w] = reinterpret_cast<const uint32_t *>(tile + tid * TILE_STRIDE)[w];
    __syncthreads();                                        // the tile is in registers: its memory becomes the image
    for (uint32_t i = tid; i * 16 < end + 4; i += ENC_THREADS) reinterpret_cast<uint4 *>(out)[i] = make_uint4(0u, 0u, 0u, 0u);
    __syncthreads();
    const uint32_t start = lead + (tid ? (uint32_t)(tinfo[tid - 1] >> 3) : 0u);
    if (long_codes) encode_vector<false>(row, tab, out, start);
    else encode_vector<true>(row, tab, out, start);
    __syncthreads();
    // image words hold stream bytes most-significant first; swap to memory order on the way out
    uint8_t *g0 = dst - lead;                                   // 16-byte aligned
    for (uint32_t ch = tid; ch * 16 < end; ch += ENC_THREADS) {
        uint32_t b0 = ch * 16, b1 = b0 + 16;
        uint4 wv = *reinterpret_cast<const uint4 *>(&out[ch * 4]);
        wv.x = kvc_bswap(wv.x); wv.y = kvc_bswap(wv.y); wv.z = kvc_bswap(wv.z); wv.w = kvc_bswap(wv.w);
        if (b0 >= lead && b1 <= end) {
            *reinterpret_cast<uint4 *>(g0 + b0) = wv;
        } else {                                                // shared with a neighbouring block
            const uint8_t *bytes = reinterpret_cast<const uint8_t *>(&wv);
            for (uint32_t b = (b0 < lead ? lead : b0); b < (b1 < end ? b1 : end); b++) g0[b] = bytes[b - b0];
        }
    }
}

}  // namespace

extern "C" int64_t kvc_encode_workspace(int64_t T, int64_t cols, int is_k) {
    int64_t nblk = is_k ? (T / 64) * cols : (T / 128) * cols * 2;
    int64_t n_part = (nblk + 1023) / 1024;
    return ((nblk * 4 + 15) / 16) * 16 + (n_part + 1) * 8;
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
    if (nblk == 0) {
        if (total_bytes) KVC_CUDA_OK(cudaMemsetAsync(total_bytes, 0, 8, s));
        return KVC_OK;
    }
    KVC_REQUIRE(nblk < (1ll << 31), "kvc_encode: too many blocks in one call");
    KVC_REQUIRE(workspace && workspace_bytes >= kvc_encode_workspace(T, cols, is_k),
                "kvc_encode: workspace needs %lld bytes", (long long)kvc_encode_workspace(T, cols, is_k));
    KVC_REQUIRE((reinterpret_cast<uintptr_t>(workspace) & 15) == 0, "kvc_encode: workspace must be 16-byte aligned");
    const long long n_part = (nblk + 1023) / 1024;
    uint32_t *sizes = reinterpret_cast<uint32_t *>(workspace);
    unsigned long long *partial = reinterpret_cast<unsigned long long *>(
        reinterpret_cast<uint8_t *>(workspace) + ((nblk * 4 + 15) / 16) * 16);
    const uint32_t *enc = reinterpret_cast<const uint32_t *>(enc_table);
    KVC_CUDA_OK(cudaMemsetAsync(partial, 0, (n_part + 1) * 8, s));
    encode_sizes_kernel<<<(unsigned)nblk, ENC_THREADS, 0, s>>>(codes, cols, is_k, enc, n_entries, thread_info, sizes, partial,
                                                      total_bytes ? total_bytes + 1 : nullptr, status);
    scan_partials_kernel<<<1, 1024, 0, s>>>(partial, n_part, total_bytes);
    scan_blocks_kernel<<<(unsigned)n_part, 1024, 0, s>>>(sizes, nblk, partial, base_offset, encoded_capacity,
                                                        reinterpret_cast<uint2 *>(block_info), status);
    encode_emit_kernel<<<(unsigned)nblk, ENC_THREADS, 0, s>>>(codes, cols, is_k, enc, n_entries, thread_info,
                                                     reinterpret_cast<const uint2 *>(block_info), sizes, base_offset,
                                                     encoded, encoded_capacity);
    KVC_LAUNCH_OK();
    return KVC_OK;
}
