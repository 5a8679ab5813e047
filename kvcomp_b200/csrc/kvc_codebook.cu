// 256-bin symbol histogram and the Huffman codebook build, on the device.
//
// The code assignment reproduces src/huffman.cpp:34-96 (== utils/huffman.py:47-81) bit for
// bit: leaves pushed in ascending symbol order into a binary min-heap keyed on frequency
// only, first popped = left = '0', second popped = right = '1', root-to-leaf path codes.
// The heap discipline (which decides every tie) is the one std::priority_queue and CPython's
// heapq share: push = append + sift up while the parent is strictly larger; pop = walk the
// hole from the root to a leaf always taking the right child unless it is strictly larger
// than the left one, drop the former last element there and sift it up.
#include <stdarg.h>

#include "kvc_common.cuh"

static thread_local char g_err[512] = "";

void kvc_set_error(const char *fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_err, sizeof(g_err), fmt, ap);
    va_end(ap);
}

extern "C" const char *kvc_last_error(void) { return g_err; }
extern "C" int kvc_version(void) { return KVC_VERSION; }

int kvc_sm_count() {
    int dev = 0, n = 0;
    if (cudaGetDevice(&dev) != cudaSuccess) return 148;
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) return 148;
    return n;
}

extern "C" int kvc_buffer_sizes(int64_t tokens, int64_t hidden, int is_k, int64_t out[4]) {
    KVC_REQUIRE(out != nullptr, "kvc_buffer_sizes: out is null");
    // kernels.cu:898-909: K needs tokens % 64 == 0 and hidden % 128 == 0; V tokens % 128, hidden % 64
    if (is_k) {
        KVC_REQUIRE(tokens % KVC_VEC_PER_BLK == 0, "Context length must be divisible by K_VEC_PER_BLK");
        KVC_REQUIRE(hidden % KVC_VEC_LEN == 0, "Hidden dim must be divisible by K_VEC_LEN");
    } else {
        KVC_REQUIRE(tokens % KVC_VEC_LEN == 0, "Context length must be divisible by V_VEC_LEN");
        KVC_REQUIRE(hidden % KVC_VEC_PER_BLK == 0, "Hidden dim must be divisible by V_VEC_PER_BLK");
    }
    int64_t numel = tokens * hidden;
    out[0] = numel / KVC_VEC_LEN / KVC_VEC_PER_BLK * 8;
    out[1] = numel / KVC_VEC_LEN * 2;
    out[2] = 8;
    out[3] = numel;
    return KVC_OK;
}

namespace {

// ---- histogram: per-warp private bins in shared memory, 16 codes per load ----------------------
__global__ void __launch_bounds__(256) histogram_kernel(const uint8_t *__restrict__ codes, long long n,
                                                        unsigned long long *__restrict__ hist) {
    __shared__ unsigned int sh[8][256];
    const int tid = threadIdx.x, warp = tid >> 5;
    for (int i = tid; i < 8 * 256; i += 256) (&sh[0][0])[i] = 0;
    __syncthreads();
    const long long head = ((16 - (reinterpret_cast<uintptr_t>(codes) & 15)) & 15);   // bytes before alignment
    const long long pre = head < n ? head : n;
    const long long nvec = (n - pre) / 16;
    const uint4 *v = reinterpret_cast<const uint4 *>(codes + pre);
    for (long long i = (long long)blockIdx.x * 256 + tid; i < nvec; i += (long long)gridDim.x * 256) {
        uint4 w = v[i];
        const uint8_t *b = reinterpret_cast<const uint8_t *>(&w);
#pragma unroll
        for (int k = 0; k < 16; k++) atomicAdd(&sh[warp][b[k]], 1u);
    }
    if (blockIdx.x == 0) {   // unaligned head and the tail shorter than 16
        for (long long i = tid; i < pre; i += 256) atomicAdd(&sh[warp][codes[i]], 1u);
        for (long long i = pre + nvec * 16 + tid; i < n; i += 256) atomicAdd(&sh[warp][codes[i]], 1u);
    }
    __syncthreads();
    unsigned int s = 0;
#pragma unroll
    for (int w = 0; w < 8; w++) s += sh[w][tid];
    if (s) atomicAdd(&hist[tid], (unsigned long long)s);
}

// ---- heap, exactly as described at the top of the file -----------------------------------------
// A node is one 64-bit word, (frequency << 10) | id, so that a move in the heap is one load and one
// store; comparisons look at the frequency alone, as the reference's do (ties are decided by position).
struct Heap { unsigned long long *w; int n; };
__device__ __forceinline__ unsigned long long heap_word(long long f, short id) { return ((unsigned long long)f << 10) | (unsigned long long)(id & 0x3ff); }
__device__ __forceinline__ unsigned long long heap_freq(unsigned long long w) { return w >> 10; }

__device__ void heap_sift_up(Heap &hp, int hole, unsigned long long word) {
    while (hole > 0) {
        const int parent = (hole - 1) >> 1;
        const unsigned long long pw = hp.w[parent];
        if (!(heap_freq(pw) > heap_freq(word))) break;
        hp.w[hole] = pw;
        hole = parent;
    }
    hp.w[hole] = word;
}
__device__ void heap_push(Heap &hp, long long f, short id) { hp.n++; heap_sift_up(hp, hp.n - 1, heap_word(f, id)); }
__device__ short heap_pop(Heap &hp, long long *f_out) {
    const unsigned long long top = hp.w[0];
    *f_out = (long long)heap_freq(top);
    const short top_id = (short)(top & 0x3ff);
    int len = --hp.n;
    if (len == 0) return top_id;
    const unsigned long long last = hp.w[len];
    int hole = 0, child = 0;
    while (child < (len - 1) / 2) {
        child = 2 * (child + 1);
        unsigned long long c1 = hp.w[child], c0 = hp.w[child - 1];
        if (heap_freq(c1) > heap_freq(c0)) { child--; c1 = c0; }
        hp.w[hole] = c1;
        hole = child;
    }
    if ((len & 1) == 0 && child == (len - 2) / 2) {
        child = 2 * (child + 1);
        hp.w[hole] = hp.w[child - 1];
        hole = child - 1;
    }
    heap_sift_up(hp, hole, last);
    return top_id;
}

struct BookSmem {
    long long hf[512];
    short hid[512];
    short left[512], right[512];
    uint32_t enc_code[256], enc_len[256];
    uint32_t tree[512];          // wide tree: lo16 = child0 (or LEAF), hi16 = child1 (or symbol)
    long long count[256];        // the histogram, fetched by all threads at once
    int n_nodes, n_symbols, min_sym, max_sym, max_len, flags;
};

// insert every code into the decode trees in ascending symbol order
// (build_decode_code_book, src/huffman.cpp:229-252); run by one thread
__device__ void build_trees(BookSmem &s) {      // s.tree was cleared to {NONE, NONE} by the whole CTA
    int n = 2;
    for (int sym = 0; sym < 256; sym++) {
        int len = (int)s.enc_len[sym];
        if (!len) continue;
        int idx = -1, last = -1;
        for (int k = len - 1; k >= 0; k--) {
            int bit = (s.enc_code[sym] >> k) & 1;
            if (idx == -1) idx = bit;
            else {
                uint32_t ch = (s.tree[idx] >> (16 * bit)) & 0xffffu;
                idx = ch == KVC_TREE_NONE ? -1 : (int)ch;
            }
            if (idx == -1) {
                if (n >= 512) { s.flags |= KVC_FLAG_CODE_TOO_LONG; break; }
                uint32_t m = 0xffffu << (16 * bit);
                s.tree[last] = (s.tree[last] & ~m) | ((uint32_t)n << (16 * bit));
                idx = n++;
            }
            last = idx;
        }
        if (idx >= 0) s.tree[idx] = KVC_TREE_LEAF | ((uint32_t)sym << 16);
    }
    s.n_nodes = n;
}

// Decode table entry for a KVC_LUT_BITS-bit window w (first stream bit = MSB), 32 bits:
//   byte 0      how far the decoder state advances: (symbols << 6) | bits consumed   (0 = escape)
//   bytes 1..3  up to three complete symbols found in the window, unused bytes 0
// The decoder state is (position in the vector << 6) | bit offset, so one add applies an entry.
// When no code completes inside the window (a code longer than the window, or no code at all)
// byte 0 is 0 and the upper bytes hold the wide-tree node the window's bits lead to; the slow path
// continues from there one bit at a time.
__device__ uint32_t lut_entry(const uint32_t *tree, uint32_t w) {
    uint32_t syms = 0, nsym = 0, used = 0;
    int idx = -1, pos = 0;
    while (pos < KVC_LUT_BITS) {
        int bit = (w >> (KVC_LUT_BITS - 1 - pos)) & 1;
        uint32_t ch = idx == -1 ? (uint32_t)bit : ((tree[idx] >> (16 * bit)) & 0xffffu);
        pos++;
        if (ch == KVC_TREE_NONE || ch >= 512) { idx = -2; break; }     // no such code
        idx = (int)ch;
        if ((tree[idx] & 0xffffu) == KVC_TREE_LEAF) {
            syms |= (tree[idx] >> 16) << (8 * nsym);
            nsym++; used = pos; idx = -1;
            if (nsym == 3) break;
        }
    }
    if (nsym) return (syms << 8) | (nsym << 6) | used;
    return (idx < 0 ? (uint32_t)KVC_TREE_NONE : (uint32_t)idx) << 8;
}

__device__ void write_book(const BookSmem &s, uint8_t *book, int tid, int nthr) {
    uint32_t *enc = reinterpret_cast<uint32_t *>(book + KVC_BOOK_OFF_ENC);
    for (int i = tid; i < 256; i += nthr) { enc[2 * i] = s.enc_code[i]; enc[2 * i + 1] = s.enc_len[i]; }
    // reference-format tree: {u8 is_leaf, i8 a, i8 b}; indices and symbols narrowed to 8 bits as
    // include/huffman.h:18-22 does, unset child = -1
    uint8_t *rt = book + KVC_BOOK_OFF_REFTREE;
    for (int i = tid; i < 512; i += nthr) {
        uint32_t nd = s.tree[i];
        uint8_t leaf = 0, a = 0, b = 0;
        if (i < s.n_nodes) {
            if ((nd & 0xffffu) == KVC_TREE_LEAF) { leaf = 1; a = b = (uint8_t)(nd >> 16); }
            else {
                uint32_t c0 = nd & 0xffffu, c1 = nd >> 16;
                a = c0 == KVC_TREE_NONE ? 0xff : (uint8_t)c0;
                b = c1 == KVC_TREE_NONE ? 0xff : (uint8_t)c1;
            }
        }
        rt[3 * i] = leaf; rt[3 * i + 1] = a; rt[3 * i + 2] = b;
    }
    uint32_t *wt = reinterpret_cast<uint32_t *>(book + KVC_BOOK_OFF_TREE);
    for (int i = tid; i < 512; i += nthr) wt[i] = s.tree[i];
    uint32_t *lut = reinterpret_cast<uint32_t *>(book + KVC_BOOK_OFF_LUT);
    int no_code = 0;                                        // an entry whose window holds no complete code
    for (int w = tid; w < KVC_LUT_SIZE; w += nthr) {
        const uint32_t e = lut_entry(s.tree, (uint32_t)w);
        lut[w] = e;
        no_code |= (e & 0xffu) == 0;
    }
    no_code = __syncthreads_or(no_code);
    if (tid == 0) {
        kvc_book_header *h = reinterpret_cast<kvc_book_header *>(book);
        h->n_symbols = s.n_symbols; h->min_sym = s.min_sym; h->max_sym = s.max_sym; h->max_len = s.max_len;
        h->n_nodes = s.n_nodes; h->flags = s.flags; h->lut_bits = KVC_LUT_BITS; h->escape = no_code ? 1 : 0;
    }
}

__global__ void __launch_bounds__(256) build_codebook_kernel(const unsigned long long *__restrict__ hist,
                                                             uint8_t *__restrict__ book) {
    __shared__ BookSmem s;
    const int tid = threadIdx.x;
    s.enc_code[tid] = 0; s.enc_len[tid] = 0;
    s.count[tid] = (long long)hist[tid];                    // one coalesced load instead of 256 dependent ones
    s.tree[tid] = s.tree[tid + 256] = KVC_TREE_NONE | (KVC_TREE_NONE << 16);
    __syncthreads();
    if (tid == 0) {
        Heap hp; hp.w = reinterpret_cast<unsigned long long *>(s.hf); hp.n = 0;
        int nsym = 0, mn = 256, mx = -1;
        s.flags = 0;
        for (int i = 0; i < 256; i++) {
            long long c = s.count[i];
            if (c > 0) { heap_push(hp, c, (short)i); nsym++; if (i < mn) mn = i; mx = i; }
        }
        s.n_symbols = nsym; s.min_sym = nsym ? mn : 0; s.max_sym = nsym ? mx : 0; s.max_len = 0;
        if (nsym == 0) s.flags |= KVC_FLAG_NO_SYMBOLS;
        else if (nsym == 1) {          // utils/huffman.py:42-44: the lone symbol gets '0'
            const int lone = (int)(hp.w[0] & 0x3ff);
            s.enc_code[lone] = 0; s.enc_len[lone] = 1; s.max_len = 1;
        } else {
            short next = 256;
            while (hp.n > 1) {
                long long fa, fb;
                short a = heap_pop(hp, &fa);
                short b = heap_pop(hp, &fb);
                s.left[next] = a; s.right[next] = b;
                heap_push(hp, fa + fb, next);
                next++;
            }
            // iterative walk; the heap arrays are free now and serve as the stack
            short *st_node = s.hid; long long *st_code = s.hf;     // code | (len << 40)
            int sp = 1;
            st_node[0] = (short)(hp.w[0] & 0x3ff); st_code[0] = 0;
            while (sp) {
                sp--;
                short nd = st_node[sp];
                unsigned long long cl = (unsigned long long)st_code[sp];
                unsigned long long code = cl & 0xffffffffffull, len = cl >> 40;
                if (nd < 256) {
                    if (len > 32) s.flags |= KVC_FLAG_CODE_TOO_LONG;
                    s.enc_code[nd] = (uint32_t)code; s.enc_len[nd] = (uint32_t)len;
                    if ((int)len > s.max_len) s.max_len = (int)len;
                } else {
                    st_node[sp] = s.right[nd]; st_code[sp] = (long long)((((code << 1) | 1) & 0xffffffffffull) | ((len + 1) << 40)); sp++;
                    st_node[sp] = s.left[nd];  st_code[sp] = (long long)(((code << 1) & 0xffffffffffull) | ((len + 1) << 40)); sp++;
                }
            }
        }
        build_trees(s);
    }
    __syncthreads();
    write_book(s, book, tid, 256);
}

// A reference-format decode tensor (3-byte nodes; child bytes read as unsigned, 0xff = unset)
// -> the same book.  Codes are recovered by walking the tree from both root children.
__global__ void __launch_bounds__(256) book_from_tree_kernel(const uint8_t *__restrict__ rt, int n_nodes,
                                                             uint8_t *__restrict__ book) {
    __shared__ BookSmem s;
    const int tid = threadIdx.x;
    s.enc_code[tid] = 0; s.enc_len[tid] = 0;
    s.tree[tid] = s.tree[tid + 256] = KVC_TREE_NONE | (KVC_TREE_NONE << 16);
    __syncthreads();
    if (tid == 0) {
        s.flags = 0; s.max_len = 0;
        int nsym = 0, mn = 256, mx = -1;
        short *st_node = s.hid; long long *st_code = s.hf;
        int sp = 0;
        if (n_nodes >= 2) { st_node[sp] = 1; st_code[sp] = 1 | (1ll << 40); sp++; st_node[sp] = 0; st_code[sp] = 0 | (1ll << 40); sp++; }
        int guard = 0;
        while (sp && guard++ < 2048) {
            sp--;
            int nd = st_node[sp];
            unsigned long long cl = (unsigned long long)st_code[sp];
            unsigned long long code = cl & 0xffffffffffull, len = cl >> 40;
            if (nd >= n_nodes) continue;
            if (rt[3 * nd]) {
                int sym = rt[3 * nd + 1];
                if (len > 32) s.flags |= KVC_FLAG_CODE_TOO_LONG;
                s.enc_code[sym] = (uint32_t)code; s.enc_len[sym] = (uint32_t)len;
                if ((int)len > s.max_len) s.max_len = (int)len;
                nsym++; if (sym < mn) mn = sym; if (sym > mx) mx = sym;
            } else {
                int c0 = rt[3 * nd + 1], c1 = rt[3 * nd + 2];
                if (c1 != 0xff && sp < 510) { st_node[sp] = (short)c1; st_code[sp] = (long long)((((code << 1) | 1) & 0xffffffffffull) | ((len + 1) << 40)); sp++; }
                if (c0 != 0xff && sp < 510) { st_node[sp] = (short)c0; st_code[sp] = (long long)(((code << 1) & 0xffffffffffull) | ((len + 1) << 40)); sp++; }
            }
        }
        s.n_symbols = nsym; s.min_sym = nsym ? mn : 0; s.max_sym = nsym ? mx : 0;
        if (nsym == 0) s.flags |= KVC_FLAG_NO_SYMBOLS;
        build_trees(s);
    }
    __syncthreads();
    write_book(s, book, tid, 256);
}

}  // namespace

extern "C" int kvc_histogram(const uint8_t *codes, int64_t n, unsigned long long *hist, kvc_stream_t stream) {
    KVC_REQUIRE(hist != nullptr && (codes != nullptr || n == 0), "kvc_histogram: null pointer");
    KVC_REQUIRE(n >= 0, "kvc_histogram: negative length");
    if (n == 0) return KVC_OK;
    long long want = (n / 16 + 255) / 256;
    long long cap = (long long)kvc_sm_count() * 8;
    unsigned grid = (unsigned)(want < 1 ? 1 : (want > cap ? cap : want));
    histogram_kernel<<<grid, 256, 0, kvc_cu(stream)>>>(codes, n, hist);
    KVC_LAUNCH_OK();
    return KVC_OK;
}

extern "C" int kvc_build_codebook(const unsigned long long *hist, void *book, kvc_stream_t stream) {
    KVC_REQUIRE(hist && book, "kvc_build_codebook: null pointer");
    KVC_REQUIRE((reinterpret_cast<uintptr_t>(book) & 15) == 0, "kvc_build_codebook: book must be 16-byte aligned");
    build_codebook_kernel<<<1, 256, 0, kvc_cu(stream)>>>(hist, reinterpret_cast<uint8_t *>(book));
    KVC_LAUNCH_OK();
    return KVC_OK;
}

extern "C" int kvc_book_from_tree(const uint8_t *ref_tree, int64_t tree_bytes, void *book, kvc_stream_t stream) {
    KVC_REQUIRE(ref_tree && book, "kvc_book_from_tree: null pointer");
    KVC_REQUIRE(tree_bytes % 3 == 0 && tree_bytes >= 6, "kvc_book_from_tree: a decode tensor holds 3-byte nodes, at least two");
    KVC_REQUIRE(tree_bytes / 3 <= 255, "kvc_book_from_tree: %lld nodes; 8-bit child indices address at most 255", (long long)(tree_bytes / 3));
    KVC_REQUIRE((reinterpret_cast<uintptr_t>(book) & 15) == 0, "kvc_book_from_tree: book must be 16-byte aligned");
    book_from_tree_kernel<<<1, 256, 0, kvc_cu(stream)>>>(ref_tree, (int)(tree_bytes / 3), reinterpret_cast<uint8_t *>(book));
    KVC_LAUNCH_OK();
    return KVC_OK;
}
