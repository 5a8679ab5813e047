// Blocked Huffman decoder to uint8 codes (kernels.cu:602-719 restated for sm_100a).
//
// CTA = 256 threads = 4 blocks of 64 vectors per round, grid-stride over block groups so that the
// decode table is brought into shared memory once per CTA.  Thread = one vector; decoded symbols
// go to a shared-memory tile and leave as coalesced 32-bit stores (K: rows, V: transposed back).
#include "kvc_decode.cuh"

namespace {

constexpr int TILE_STRIDE = 140;          // 128 symbols + KVC_DECODE_OVERRUN_PAIR rounded up to words, + 1 word; 35 words keep column reads off one bank

struct DecodeSmem {                         // followed by 4 staging slots (sized at launch), then the 4 tiles
    KvcBookSmem book;
};
constexpr int TILE_BYTES = 64 * TILE_STRIDE; // a tile; the tiles are also the padding a corrupt stream's overrun reads land in

__global__ void __launch_bounds__(256) decode_kernel(
    const uint8_t *__restrict__ encoded, long long encoded_bytes, const uint2 *__restrict__ block_info,
    const uint16_t *__restrict__ thread_info, const void *__restrict__ book, long long nblk, long long cols, int is_k,
    uint32_t max_block, uint32_t slot_bytes, uint8_t *__restrict__ codes, int *__restrict__ status) {
    extern __shared__ __align__(16) uint8_t smem_raw[];
    DecodeSmem &sm = *reinterpret_cast<DecodeSmem *>(smem_raw);
    uint8_t *const slots = smem_raw + sizeof(DecodeSmem), *const tiles = slots + 4 * slot_bytes;
    const bool esc = kvc_book_needs_escape(book);           // uniform over the grid
    const int tid = threadIdx.x, sub = tid >> 6, v = tid & 63;      // sub-block and vector of this thread
    const long long row = cols * 128;
    kvc_load_book(sm.book, book, tid, 256);
    int flags = 0;
    for (long long grp = blockIdx.x; grp * 4 < nblk; grp += gridDim.x) {
        const long long blk = grp * 4 + sub;
        const bool active = blk < nblk;
        uint32_t lead = 0, nbytes = 0;
        __syncthreads();                       // previous round's tile and slot are free (and the book is in)
        if (active) {
            const uint2 bi = block_info[blk];
            nbytes = bi.y & 0xffffu;
            if (nbytes > max_block || (long long)bi.x + nbytes > encoded_bytes) { nbytes = 0; flags |= KVC_FLAG_BAD_STREAM; }
            lead = kvc_stage_block(slots + sub * slot_bytes, encoded, encoded_bytes, bi.x, nbytes, v, 64);
        }
        __syncthreads();
        if (active && nbytes) {
            const uint32_t start = v ? (uint32_t)(thread_info[blk * 64 + v - 1] >> 3) : 0u;
            uint8_t *trow = tiles + sub * TILE_BYTES + v * TILE_STRIDE;
            bool ok = start < nbytes;
            // the symbols of the lookups collect in a register pair and leave as whole words; symbols
            // past position 127 (at most KVC_DECODE_OVERRUN_PAIR) land in the row's padding words
            unsigned long long buf = 0;
            uint32_t fill = 0;                               // bytes held in buf, < 4 between lookups
            uint32_t *wrow = reinterpret_cast<uint32_t *>(trow);
            auto put = [&](uint32_t e, uint32_t) {
                buf |= (unsigned long long)(e >> 8) << (fill * 8);
                fill += (e >> 6) & 3u;
                if (fill >= 4u) { *wrow++ = (uint32_t)buf; buf >>= 32; fill -= 4u; }
            };
            const uint32_t slot_s = kvc_smem_addr(slots + sub * slot_bytes), lut_s = kvc_smem_addr(sm.book.lut),
                           tree_s = kvc_smem_addr(sm.book.tree);
            if (ok) ok = esc ? kvc_decode_vector<true, 0>(slot_s, lead + start, lut_s, tree_s, 0u, put)
                             : kvc_decode_vector<false, 0, decltype(put), true>(slot_s, lead + start, lut_s, tree_s, 0u, put);
            if (ok && wrow < reinterpret_cast<uint32_t *>(trow) + TILE_STRIDE / 4) *wrow = (uint32_t)buf;
            if (!ok) flags |= KVC_FLAG_BAD_STREAM;
        }
        __syncthreads();
        if (active && nbytes) {
            const uint8_t *tile = tiles + sub * TILE_BYTES;
            if (is_k) {
                const long long j = blk / cols, col = blk % cols;
                uint8_t *dst = codes + (j * 64) * row + col * 128;
                if ((reinterpret_cast<uintptr_t>(codes) & 15) == 0) {
#pragma unroll
                    for (int k = 0; k < 8; k++) {            // 64 rows x 8 chunks of 16 bytes
                        const int i = v + k * 64, r = i >> 3, c = i & 7;
                        const uint32_t *t4 = reinterpret_cast<const uint32_t *>(tile + r * TILE_STRIDE + c * 16);
                        *reinterpret_cast<uint4 *>(dst + r * row + c * 16) = make_uint4(t4[0], t4[1], t4[2], t4[3]);
                    }
                } else {
                    for (int i = v; i < 64 * 32; i += 64) {
                        int r = i >> 5, w = i & 31;
                        *reinterpret_cast<uint32_t *>(dst + r * row + w * 4) =
                            *reinterpret_cast<const uint32_t *>(tile + r * TILE_STRIDE + w * 4);
                    }
                }
            } else {
                const long long g = blk / (cols * 2), m = blk % (cols * 2);
                uint8_t *dst = codes + (g * 128) * row + m * 64;
                for (int i = v; i < 32 * 16; i += 64) {     // 32 groups of 4 tokens x 16 words of 4 channels
                    const int tg = i >> 4, w = i & 15;
                    uint32_t x0 = *reinterpret_cast<const uint32_t *>(tile + (w * 4 + 0) * TILE_STRIDE + tg * 4);
                    uint32_t x1 = *reinterpret_cast<const uint32_t *>(tile + (w * 4 + 1) * TILE_STRIDE + tg * 4);
                    uint32_t x2 = *reinterpret_cast<const uint32_t *>(tile + (w * 4 + 2) * TILE_STRIDE + tg * 4);
                    uint32_t x3 = *reinterpret_cast<const uint32_t *>(tile + (w * 4 + 3) * TILE_STRIDE + tg * 4);
                    kvc_transpose4x4(x0, x1, x2, x3);          // now one word per token: its 4 channels
                    *reinterpret_cast<uint32_t *>(dst + (tg * 4 + 0) * row + w * 4) = x0;
                    *reinterpret_cast<uint32_t *>(dst + (tg * 4 + 1) * row + w * 4) = x1;
                    *reinterpret_cast<uint32_t *>(dst + (tg * 4 + 2) * row + w * 4) = x2;
                    *reinterpret_cast<uint32_t *>(dst + (tg * 4 + 3) * row + w * 4) = x3;
                }
            }
        }
    }
    if (flags) atomicOr(status, flags);
}

}  // namespace

extern "C" int kvc_decode_bounded(const uint8_t *encoded, int64_t encoded_bytes, const void *block_info,
                                  const uint16_t *thread_info, const void *book, int64_t T, int64_t cols, int is_k,
                                  uint32_t max_block_bytes, uint8_t *codes, int32_t *status, kvc_stream_t stream) {
    KVC_REQUIRE(encoded && block_info && thread_info && book && codes && status, "kvc_decode: null pointer");
    KVC_REQUIRE(cols > 0 && T >= 0 && encoded_bytes >= 0, "kvc_decode: bad shape");
    KVC_REQUIRE(T % (is_k ? 64 : 128) == 0, "kvc_decode: %s needs a multiple of %d tokens, got %lld",
                is_k ? "K" : "V", is_k ? 64 : 128, (long long)T);
    KVC_REQUIRE((reinterpret_cast<uintptr_t>(codes) & 3) == 0 && (reinterpret_cast<uintptr_t>(block_info) & 7) == 0 &&
                (reinterpret_cast<uintptr_t>(book) & 15) == 0, "kvc_decode: misaligned pointer");
    const long long nblk = is_k ? (T / 64) * cols : (T / 128) * cols * 2;
    if (nblk == 0) return KVC_OK;
    // a slot holds the largest block plus its alignment lead, in 16-byte chunks, plus the decoder's read-ahead
    const uint32_t max_block = max_block_bytes == 0 || max_block_bytes > 8191u ? 8191u : max_block_bytes;
    const uint32_t slot_bytes = ((max_block + 15u + 15u) & ~15u) + 16u;
    const size_t smem = sizeof(DecodeSmem) + 4 * (size_t)slot_bytes + 4 * (size_t)TILE_BYTES;
    KVC_CUDA_OK(cudaFuncSetAttribute(decode_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    KVC_CUDA_OK(cudaFuncSetAttribute(decode_kernel, cudaFuncAttributePreferredSharedMemoryCarveout, 100));
    int occ = 0;
    KVC_CUDA_OK(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&occ, decode_kernel, 256, smem));
    KVC_REQUIRE(occ >= 1, "kvc_decode: %zu bytes of shared memory do not fit an SM", smem);
    long long groups = (nblk + 3) / 4, cap = (long long)kvc_sm_count() * occ;
    unsigned grid = (unsigned)(groups < cap ? groups : cap);
    decode_kernel<<<grid, 256, smem, kvc_cu(stream)>>>(
        encoded, encoded_bytes, reinterpret_cast<const uint2 *>(block_info), thread_info, book, nblk, cols, is_k,
        max_block, slot_bytes, codes, status);
    KVC_LAUNCH_OK();
    return KVC_OK;
}

extern "C" int kvc_decode(const uint8_t *encoded, int64_t encoded_bytes, const void *block_info,
                          const uint16_t *thread_info, const void *book, int64_t T, int64_t cols, int is_k,
                          uint8_t *codes, int32_t *status, kvc_stream_t stream) {
    return kvc_decode_bounded(encoded, encoded_bytes, block_info, thread_info, book, T, cols, is_k, 0u, codes, status, stream);
}
