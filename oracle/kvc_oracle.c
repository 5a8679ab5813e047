/*
 * CPU restatement of the KVComp hot path -- TEST INFRASTRUCTURE ONLY.
 *
 * This file is a checker.  It restates, in plain C, the algorithm of the
 * reference's KV-cache compression path so that the CUDA library can be compared
 * against it bit for bit.  Nothing in the product (the kvcomp_b200 package or
 * libkvcomp_b200.so) may link, import or call it; only the test-suite, the smoke
 * entry and the cpu_baseline / reference arm of the benchmark do.
 *
 * Parity pin: the quantiser and the code assignment are pinned against golden
 * vectors generated from the reference's own Python path (utils/compute.py,
 * utils/huffman.py) and from the reference's own src/huffman.cpp compiled as is;
 * the blocked stream layout follows kernels.cu and is pinned by round trips and
 * by the flat bit count of utils/huffman.py (see tests/test_oracle_golden.py).
 *
 * Each function cites the reference file:line it follows (paths relative to the
 * reference project root).
 */
#include <stdint.h>
#include <stdlib.h>
#include <string.h>
#include <math.h>

#ifdef _OPENMP
#include <omp.h>
#endif

/* ------------------------------------------------------------------ fp16 -- */
/* torch evaluates every fp16 elementwise op as: widen to fp32, compute, round
 * to nearest-even back to fp16.  _Float16 conversions in gcc are correctly
 * rounded, which is all that is needed here. */
static inline float h2f(uint16_t h) { _Float16 v; memcpy(&v, &h, 2); return (float)v; }
static inline uint16_t f2h(float f) { _Float16 v = (_Float16)f; uint16_t h; memcpy(&h, &v, 2); return h; }

int orc_num_threads(void) {
#ifdef _OPENMP
    return omp_get_max_threads();
#else
    return 1;
#endif
}

/* --------------------------------------------------------------- quantiser -- */
/* Quant-unit addressing shared by every function below: the unit that element
 * (t, b, h, c) of a token-major [T,B,H,D] tensor belongs to is
 *     (t / tok_div) * sj + b * sb + h * sh + c * sc
 * with a stride of zero for every dimension the unit spans. */
typedef struct { int64_t tok_div, sj, sb, sh, sc; } orc_qmeta;

enum { ORC_MODE_BLOCK = 0, ORC_MODE_CHANNEL = 1, ORC_MODE_TOKEN = 2, ORC_MODE_VECTOR = 3 };

/* Unit shapes.  batch_shared = 1 follows the reference's CUDA-path tables
 * (models/cache/kvcomp_encode.py:10-13, dims [1,2,3,4] / [2,3,4] on
 * [nblk,blk,B,H,D]: the unit spans the batch); batch_shared = 0 follows
 * utils/compute.py:138-143 (dims on [B,H,nblk,blk,D]: the batch is kept).
 * Returns the number of units and fills m. */
int64_t orc_qmeta_make(int mode, int batch_shared, int64_t T, int64_t B, int64_t H, int64_t D,
                       int64_t block, orc_qmeta *m) {
    int64_t nb = batch_shared ? 1 : B;
    memset(m, 0, sizeof(*m));
    switch (mode) {
    case ORC_MODE_BLOCK:   /* one unit per token block (and sequence) */
        m->tok_div = block; m->sj = nb; m->sb = batch_shared ? 0 : 1;
        return (T / block) * nb;
    case ORC_MODE_CHANNEL: /* utils/compute.py:140, one unit per (block, b, h, channel) */
        m->tok_div = block; m->sj = B * H * D; m->sb = H * D; m->sh = D; m->sc = 1;
        return (T / block) * B * H * D;
    case ORC_MODE_TOKEN:   /* one unit per token (and sequence) */
        m->tok_div = 1; m->sj = nb; m->sb = batch_shared ? 0 : 1;
        return T * nb;
    case ORC_MODE_VECTOR:  /* utils/compute.py:142, one unit per (token, b, h) */
        m->tok_div = 1; m->sj = B * H; m->sb = H; m->sh = 1;
        return T * B * H;
    }
    return -1;
}

/* utils/compute.py:93-106 (quant) and :74-91 (quant_ints); C++ twin
 * src/compute.cpp:40-58.  fp16 tensor arithmetic, every op rounded:
 *   scale   = fp16( fp32(fp16(max - min)) * fp32(rel) )
 *   min_int = rint( fp16( min / scale ) )
 *   code    = fp16( rint(fp16(x / scale)) - min_int )
 * codes -> uint8 as models/cache/kvcomp_encode.py:98.  min_int is returned as int16, i.e.
 * exactly; the reference narrows it to int8 (kvcomp_encode.py:97), which wraps when
 * |min/scale| > 127 (small rel, data far from zero) -- callers that want the reference's
 * stored value narrow it themselves.
 * code_f (optional) receives the un-narrowed fp16 code values, min_f the
 * un-narrowed fp16 min_int, so that narrowing overflow can be seen by a test.
 * A unit whose scale is zero (constant input) yields NaN in the reference; here
 * its codes and min_int are written as 0 and the return value counts such units. */
int64_t orc_quant(const uint16_t *x, int64_t T, int64_t B, int64_t H, int64_t D,
                  int mode, int batch_shared, int64_t block, float rel,
                  uint8_t *codes, int16_t *min_int, uint16_t *scale,
                  uint16_t *code_f, uint16_t *min_f) {
    orc_qmeta m;
    int64_t nunit = orc_qmeta_make(mode, batch_shared, T, B, H, D, block, &m);
    if (nunit < 0) return -1;
    float *mn = (float *)malloc(sizeof(float) * nunit);
    float *mx = (float *)malloc(sizeof(float) * nunit);
    float *mi = (float *)malloc(sizeof(float) * nunit);
    for (int64_t u = 0; u < nunit; u++) { mn[u] = INFINITY; mx[u] = -INFINITY; }
    for (int64_t t = 0; t < T; t++)
        for (int64_t b = 0; b < B; b++)
            for (int64_t h = 0; h < H; h++) {
                const uint16_t *row = x + ((t * B + b) * H + h) * D;
                int64_t ub = (t / m.tok_div) * m.sj + b * m.sb + h * m.sh;
                for (int64_t c = 0; c < D; c++) {
                    float v = h2f(row[c]);
                    int64_t u = ub + c * m.sc;
                    if (v < mn[u]) mn[u] = v;
                    if (v > mx[u]) mx[u] = v;
                }
            }
    int64_t degenerate = 0;
    for (int64_t u = 0; u < nunit; u++) {
        float range = h2f(f2h(mx[u] - mn[u]));
        uint16_t s = f2h(range * rel);
        scale[u] = s;
        float sf = h2f(s);
        if (sf == 0.0f || sf != sf) { mi[u] = 0.0f; degenerate++; }
        else mi[u] = nearbyintf(h2f(f2h(mn[u] / sf)));
        if (min_f) min_f[u] = f2h(mi[u]);
        min_int[u] = (int16_t)(int)mi[u];
    }
#pragma omp parallel for schedule(static)
    for (int64_t t = 0; t < T; t++)
        for (int64_t b = 0; b < B; b++)
            for (int64_t h = 0; h < H; h++) {
                int64_t base = ((t * B + b) * H + h) * D;
                int64_t ub = (t / m.tok_div) * m.sj + b * m.sb + h * m.sh;
                for (int64_t c = 0; c < D; c++) {
                    int64_t u = ub + c * m.sc;
                    float sf = h2f(scale[u]);
                    float cf;
                    if (sf == 0.0f || sf != sf) cf = 0.0f;
                    else {
                        float q = nearbyintf(h2f(f2h(h2f(x[base + c]) / sf)));
                        cf = h2f(f2h(q - mi[u]));
                    }
                    if (code_f) code_f[base + c] = f2h(cf);
                    codes[base + c] = (uint8_t)(int)cf;
                }
            }
    free(mn); free(mx); free(mi);
    return degenerate;
}

/* models/cache/kvcomp_encode.py:146 and utils/compute.py:130:
 * x^ = fp16( fp16(code + min_int) * scale ), the sum being exact in fp16. */
void orc_dequant(const uint8_t *codes, const int16_t *min_int, const uint16_t *scale,
                 int64_t T, int64_t B, int64_t H, int64_t D, const orc_qmeta *m, uint16_t *out) {
#pragma omp parallel for schedule(static)
    for (int64_t t = 0; t < T; t++)
        for (int64_t b = 0; b < B; b++)
            for (int64_t h = 0; h < H; h++) {
                int64_t base = ((t * B + b) * H + h) * D;
                int64_t ub = (t / m->tok_div) * m->sj + b * m->sb + h * m->sh;
                for (int64_t c = 0; c < D; c++) {
                    int64_t u = ub + c * m->sc;
                    float s = h2f(f2h((float)((int)codes[base + c] + (int)min_int[u])));
                    out[base + c] = f2h(s * h2f(scale[u]));
                }
            }
}

/* utils/compute.py:59-72 (cut_tensor_ctx_len_0) / :44-57: number of leading
 * tokens that get compressed when `len` tokens are buffered. */
int64_t orc_cut_len(int64_t len, int64_t block, int64_t recent) {
    int64_t num = len + block - len % block - recent;   /* may be negative: nothing to cut */
    int64_t n = num >= block ? (num / block) * block : 0;
    return n > len ? len : n;   /* the slice clips: with recent = 0 the count overshoots by one block */
}

/* ----------------------------------------------------- histogram, codebook -- */
/* src/huffman.cpp:105-109: one 256-bin histogram over every code of the call. */
void orc_histogram(const uint8_t *codes, int64_t n, int64_t *counts /*[256], accumulated*/) {
    for (int64_t i = 0; i < n; i++) counts[codes[i]]++;
}

typedef struct { uint32_t code, length; } orc_enc;   /* include/huffman.h:13-16 */

/* Binary min-heap on frequency exactly as std::priority_queue<.., CompareNodes>
 * (src/huffman.cpp:22-26,37,41-57) and CPython heapq with __lt__ on freq
 * (utils/huffman.py:12-13,47-64) order it.  push: append, sift up while the
 * parent is strictly larger.  pop: move the hole from the root to a leaf always
 * taking the right child unless it is strictly larger than the left one, drop the
 * former last element there, sift it up (strict). */
typedef struct { int64_t f[512]; int id[512]; int n; } orc_heap;

static void heap_sift_up(orc_heap *hp, int hole, int top, int64_t f, int id) {
    while (hole > top) {
        int parent = (hole - 1) / 2;
        if (!(hp->f[parent] > f)) break;
        hp->f[hole] = hp->f[parent]; hp->id[hole] = hp->id[parent];
        hole = parent;
    }
    hp->f[hole] = f; hp->id[hole] = id;
}
static void heap_push(orc_heap *hp, int64_t f, int id) { hp->n++; heap_sift_up(hp, hp->n - 1, 0, f, id); }
static int heap_pop(orc_heap *hp, int64_t *f_out) {
    int top_id = hp->id[0]; *f_out = hp->f[0];
    int len = --hp->n;                 /* elements left after removing the root */
    if (len == 0) return top_id;
    int64_t vf = hp->f[len]; int vid = hp->id[len];
    int hole = 0, child = 0;
    while (child < (len - 1) / 2) {
        child = 2 * (child + 1);                       /* right child */
        if (hp->f[child] > hp->f[child - 1]) child--;  /* right strictly larger -> left */
        hp->f[hole] = hp->f[child]; hp->id[hole] = hp->id[child];
        hole = child;
    }
    if ((len & 1) == 0 && child == (len - 2) / 2) {    /* a lone left child */
        child = 2 * (child + 1);
        hp->f[hole] = hp->f[child - 1]; hp->id[hole] = hp->id[child - 1];
        hole = child - 1;
    }
    heap_sift_up(hp, hole, 0, vf, vid);
    return top_id;
}

/* src/huffman.cpp:34-96 (gen_huffman_codes) == utils/huffman.py:47-81.
 * enc[256] is indexed by symbol; absent symbols get {0,0}.  Returns the number
 * of distinct symbols.  A single distinct symbol gets the code '0' of length 1
 * (utils/huffman.py:42-44; the C++ path crashes on it). */
int orc_gen_codes(const int64_t *counts, orc_enc *enc) {
    int left[512], right[512];
    orc_heap hp; hp.n = 0;
    int nsym = 0, next = 256;
    memset(enc, 0, sizeof(orc_enc) * 256);
    for (int i = 0; i < 256; i++)
        if (counts[i] > 0) { heap_push(&hp, counts[i], i); nsym++; left[i] = right[i] = -1; }
    if (nsym == 0) return 0;
    if (nsym == 1) { enc[hp.id[0]].code = 0; enc[hp.id[0]].length = 1; return 1; }
    while (hp.n > 1) {
        int64_t fa, fb;
        int a = heap_pop(&hp, &fa);
        int b = heap_pop(&hp, &fb);
        left[next] = a; right[next] = b;
        heap_push(&hp, fa + fb, next);
        next++;
    }
    /* root -> leaf paths: left = 0, right = 1, first branch = most significant */
    int stack_n[512]; uint32_t stack_c[512]; uint32_t stack_l[512]; int sp = 0;
    stack_n[0] = hp.id[0]; stack_c[0] = 0; stack_l[0] = 0; sp = 1;
    while (sp) {
        sp--;
        int nd = stack_n[sp]; uint32_t c = stack_c[sp], l = stack_l[sp];
        if (nd < 256) { enc[nd].code = c; enc[nd].length = l; }
        else {
            stack_n[sp] = right[nd]; stack_c[sp] = (c << 1) | 1; stack_l[sp] = l + 1; sp++;
            stack_n[sp] = left[nd];  stack_c[sp] = (c << 1);     stack_l[sp] = l + 1; sp++;
        }
    }
    return nsym;
}

/* src/huffman.cpp:166-187 + :99-157: the encode tensor holds (max-min+1)
 * little-endian {u32 code, u32 length} entries starting at the smallest present
 * symbol.  Writes them to out (capacity 256 entries) and returns the entry
 * count; *shift receives the smallest symbol. */
int orc_ref_encode_table(const orc_enc *enc, orc_enc *out, int *shift) {
    int mn = 256, mx = -1;
    for (int i = 0; i < 256; i++) if (enc[i].length) { if (i < mn) mn = i; if (i > mx) mx = i; }
    if (mx < 0) { *shift = 0; return 0; }
    for (int i = mn; i <= mx; i++) out[i - mn] = enc[i];
    *shift = mn;
    return mx - mn + 1;
}

/* src/huffman.cpp:229-252 (build_decode_code_book), include/huffman.h:18-22:
 * 3-byte nodes {u8 is_leaf, i8 a, i8 b}; nodes 0 and 1 are the root's 0- and
 * 1-children; symbols are inserted in ascending order, a missing child takes the
 * next node index; a leaf stores its symbol in both a and b; an unset child is
 * -1.  Child indices and symbols are narrowed to int8 exactly as the reference
 * does, so trees with more than 127 nodes come out wrapped, as they do there.
 * The walk itself uses wide indices so that construction stays well defined.
 * out capacity: 3*512 bytes.  Returns the node count. */
int orc_ref_decode_tree(const orc_enc *enc, uint8_t *out) {
    int child[512][2]; int leaf[512]; int sym[512]; int n = 2;
    for (int i = 0; i < 512; i++) { child[i][0] = child[i][1] = -1; leaf[i] = 0; sym[i] = 0; }
    for (int s = 0; s < 256; s++) {
        if (!enc[s].length) continue;
        int idx = -1, last = -1;
        for (int k = (int)enc[s].length - 1; k >= 0; k--) {
            int bit = (enc[s].code >> k) & 1;
            idx = (idx == -1) ? bit : child[idx][bit];
            if (idx == -1) { child[last][bit] = n; idx = n; n++; }
            last = idx;
        }
        leaf[idx] = 1; sym[idx] = s;
    }
    for (int i = 0; i < n; i++) {
        out[3 * i] = (uint8_t)leaf[i];
        out[3 * i + 1] = (uint8_t)(int8_t)(leaf[i] ? sym[i] : child[i][0]);
        out[3 * i + 2] = (uint8_t)(int8_t)(leaf[i] ? sym[i] : child[i][1]);
    }
    return n;
}

/* ------------------------------------------------------------ stream codec -- */
/* kernels.cu:181-235 (entropy_encode): the codes of one 128-symbol vector are
 * concatenated most-significant-bit first and zero-padded to a whole byte.
 * Symbols whose table length is 0 add nothing (the reference drops them
 * silently).  Returns the bit count; *missing counts dropped symbols. */
static int encode_vector(const orc_enc *enc, const uint8_t *sym, int64_t stride, uint8_t *out,
                         int cap, int64_t *missing) {
    uint64_t acc = 0; int nacc = 0, bits = 0, nbytes = 0;
    for (int i = 0; i < 128; i++) {
        orc_enc e = enc[sym[i * stride]];
        if (!e.length) { (*missing)++; continue; }
        for (int k = (int)e.length - 1; k >= 0; k--) {
            acc = (acc << 1) | ((e.code >> k) & 1); nacc++; bits++;
            if (nacc == 8) { if (nbytes < cap) out[nbytes] = (uint8_t)acc; nbytes++; acc = 0; nacc = 0; }
        }
    }
    if (nacc) { if (nbytes < cap) out[nbytes] = (uint8_t)(acc << (8 - nacc)); nbytes++; }
    return bits;
}

/* kernels.cu:419-489 (huffman_encode, K) and :491-596 (v_huffman_encode, V),
 * tables include/kernels.h:25-32.  Input: uint8 codes [T, cols, 128] token-major
 * (cols = B*H).
 *   K vector = the 128 channels of (token, col); K block = tokens 64j..64j+63 of
 *     one col; block id = j*cols + col.
 *   V vector = tokens 128g..128g+127 of one channel column ch in [0, cols*128);
 *     V block = 64 adjacent channel columns of group g; id = g*(cols*2) + m.
 * Block bytes = its 64 vectors' bytes back to back.
 *   thread_info[block*64+v] = (end byte of v within the block << 3) | pad bits
 *   block_info[block]       = {u32 offset in the stream incl. base, u16 bytes}
 * Blocks are laid out in ascending id (the reference's order depends on an
 * atomic cursor; any order is a valid stream, this one is deterministic).
 * block_info is written as 8-byte records (u32, u16, 2 bytes zero).
 * Returns the byte length of the segment, or -1 if enc_cap is too small.
 * overflow[0] counts vectors longer than the reference's scratch (128 B for K,
 * 256 B for V; kernels.h:15,21), overflow[1] counts symbols with no code,
 * overflow[2] counts blocks whose size does not fit the u16 fields (> 8191). */
int64_t orc_encode(const uint8_t *codes, int64_t T, int64_t cols, int is_k, const orc_enc *enc,
                   uint32_t base_offset, uint8_t *block_info, uint16_t *thread_info,
                   uint8_t *encoded, int64_t enc_cap, int64_t *overflow) {
    int64_t row = cols * 128;
    int64_t nblk = is_k ? (T / 64) * cols : (T / 128) * cols * 2;
    int64_t *bsize = (int64_t *)malloc(sizeof(int64_t) * (nblk + 1));
    uint8_t *tmp = (uint8_t *)malloc((size_t)nblk * 64 * 512);
    int64_t ov0 = 0, ov1 = 0, ov2 = 0;
#pragma omp parallel for schedule(static) reduction(+:ov0,ov1,ov2)
    for (int64_t blk = 0; blk < nblk; blk++) {
        uint8_t *bt = tmp + blk * 64 * 512;
        int64_t pos = 0;
        for (int v = 0; v < 64; v++) {
            const uint8_t *src; int64_t stride;
            if (is_k) { int64_t j = blk / cols, col = blk % cols; src = codes + (j * 64 + v) * row + col * 128; stride = 1; }
            else { int64_t g = blk / (cols * 2), m = blk % (cols * 2); src = codes + (g * 128) * row + m * 64 + v; stride = row; }
            int64_t miss = 0;
            int bits = encode_vector(enc, src, stride, bt + pos, 512, &miss);
            int nb = (bits + 7) / 8;
            if (nb > (is_k ? 128 : 256)) ov0++;
            ov1 += miss;
            pos += nb;
            thread_info[blk * 64 + v] = (uint16_t)((pos << 3) + (nb * 8 - bits));
        }
        if (pos > 8191) ov2++;
        bsize[blk] = pos;
    }
    int64_t off = 0, rc = 0;
    for (int64_t blk = 0; blk < nblk; blk++) {
        if (off + bsize[blk] > enc_cap) { rc = -1; break; }
        memcpy(encoded + off, tmp + blk * 64 * 512, (size_t)bsize[blk]);
        uint32_t o = (uint32_t)(off + base_offset); uint16_t n = (uint16_t)bsize[blk];
        memset(block_info + 8 * blk, 0, 8);
        memcpy(block_info + 8 * blk, &o, 4); memcpy(block_info + 8 * blk + 4, &n, 2);
        off += bsize[blk];
    }
    if (overflow) { overflow[0] = ov0; overflow[1] = ov1; overflow[2] = ov2; }
    free(bsize); free(tmp);
    return rc < 0 ? -1 : off;
}

/* kernels.cu:237-291 (entropy_decode): walk the code tree one bit at a time over
 * the vector's bit count and emit a symbol at every leaf.  The tree here is
 * rebuilt from the encode table with wide indices (the reference's int8 node
 * indices wrap beyond 127 nodes; the walk is otherwise the same). */
typedef struct { int child[512][2]; int leaf[512]; int sym[512]; } orc_tree;
static void tree_from_enc(const orc_enc *enc, orc_tree *tr) {
    int n = 2;
    for (int i = 0; i < 512; i++) { tr->child[i][0] = tr->child[i][1] = -1; tr->leaf[i] = 0; tr->sym[i] = 0; }
    for (int s = 0; s < 256; s++) {
        if (!enc[s].length) continue;
        int idx = -1, last = -1;
        for (int k = (int)enc[s].length - 1; k >= 0; k--) {
            int bit = (enc[s].code >> k) & 1;
            idx = (idx == -1) ? bit : tr->child[idx][bit];
            if (idx == -1) { tr->child[last][bit] = n; idx = n; n++; }
            last = idx;
        }
        tr->leaf[idx] = 1; tr->sym[idx] = s;
    }
}

/* kernels.cu:602-652 (huffman_decode) and :655-719 (v_huffman_decode): inverse of
 * orc_encode, driven by block_info / thread_info.  Vector v of a block starts at
 * thread_info[v-1] >> 3 (0 for v = 0) and holds 8*(end-start) - pad bits
 * (kernels.cu:620,635).  Writes uint8 codes [T, cols, 128].  Returns the number
 * of vectors that did not decode to exactly 128 symbols. */
int64_t orc_decode(const uint8_t *encoded, const uint8_t *block_info, const uint16_t *thread_info,
                   const orc_enc *enc, int64_t T, int64_t cols, int is_k, uint8_t *codes) {
    orc_tree *tr = (orc_tree *)malloc(sizeof(orc_tree));
    tree_from_enc(enc, tr);
    int64_t row = cols * 128;
    int64_t nblk = is_k ? (T / 64) * cols : (T / 128) * cols * 2;
    int64_t bad = 0;
#pragma omp parallel for schedule(static) reduction(+:bad)
    for (int64_t blk = 0; blk < nblk; blk++) {
        uint32_t off; memcpy(&off, block_info + 8 * blk, 4);
        const uint8_t *bp = encoded + off;
        for (int v = 0; v < 64; v++) {
            int start = v ? (thread_info[blk * 64 + v - 1] >> 3) : 0;
            int ti = thread_info[blk * 64 + v];
            int nbits = (((ti >> 3) - start) << 3) - (ti & 7);
            uint8_t *dst; int64_t stride;
            if (is_k) { int64_t j = blk / cols, col = blk % cols; dst = codes + (j * 64 + v) * row + col * 128; stride = 1; }
            else { int64_t g = blk / (cols * 2), m = blk % (cols * 2); dst = codes + (g * 128) * row + m * 64 + v; stride = row; }
            int idx = -1, w = 0;
            for (int i = 0; i < nbits; i++) {
                int bit = (bp[start + (i >> 3)] >> (7 - (i & 7))) & 1;
                idx = (idx == -1) ? bit : tr->child[idx][bit];
                if (idx < 0) break;
                if (tr->leaf[idx]) { if (w < 128) dst[w * stride] = (uint8_t)tr->sym[idx]; w++; idx = -1; }
            }
            if (w != 128) bad++;
        }
    }
    free(tr);
    return bad;
}

/* --------------------------------------------------- decode-step attention -- */
/* kernels.cu:721-776 + :293-348 (fused K): raw scores
 *     S[b, hq, t] = sum_c x^_K[t, b, hkv, c] * q[b, hq, c],  hkv = hq / (Hq/Hkv)
 * with x^ = (code + min_int) * scale.  No 1/sqrt(d), mask or softmax, as there.
 * The reference accumulates in fp16; this accumulates in double over the exact
 * product (code+min)*scale, which is what the CUDA path is held to. */
void orc_qk(const uint8_t *codes, const int16_t *min_int, const uint16_t *scale, const orc_qmeta *m,
            int64_t T, int64_t B, int64_t Hkv, int64_t Hq, int64_t D, const uint16_t *q, float *S) {
    int64_t G = Hq / Hkv;
#pragma omp parallel for collapse(2) schedule(static)
    for (int64_t b = 0; b < B; b++)
        for (int64_t hq = 0; hq < Hq; hq++) {
            int64_t h = hq / G;
            for (int64_t t = 0; t < T; t++) {
                int64_t base = ((t * B + b) * Hkv + h) * D;
                int64_t ub = (t / m->tok_div) * m->sj + b * m->sb + h * m->sh;
                double acc = 0;
                for (int64_t c = 0; c < D; c++) {
                    int64_t u = ub + c * m->sc;
                    acc += (double)((int)codes[base + c] + (int)min_int[u]) * (double)h2f(scale[u]) *
                           (double)h2f(q[(b * Hq + hq) * D + c]);
                }
                S[(b * Hq + hq) * T + t] = (float)acc;
            }
        }
}

/* The reference's own fp16 chain (kernels.cu:321): result = hadd(result, hmul(hmul(half(code + min_int),
 * scale), B[c])), one channel after the other.  nvcc may contract the outer hmul with the hadd into one
 * fp16 fma (a single rounding); `fused` selects that form, so a test can hold the reference's output to
 * whichever the compiler chose.  The exact product of two fp16 values and its sum with a third fit a
 * double, and _Float16 conversions from double are correctly rounded. */
static inline uint16_t d2h(double d) { _Float16 v = (_Float16)d; uint16_t h; memcpy(&h, &v, 2); return h; }
static inline uint16_t chain_step(uint16_t r, int value, uint16_t scale, uint16_t b, int fused) {
    uint16_t v = f2h((float)value);
    uint16_t p = f2h(h2f(v) * h2f(scale));
    if (fused) return d2h((double)h2f(p) * (double)h2f(b) + (double)h2f(r));
    p = f2h(h2f(p) * h2f(b));
    return f2h(h2f(r) + h2f(p));
}

void orc_qk_fp16chain(const uint8_t *codes, const int16_t *min_int, const uint16_t *scale, const orc_qmeta *m,
                      int64_t T, int64_t B, int64_t H, int64_t D, const uint16_t *q, uint16_t *S, int fused) {
    for (int64_t b = 0; b < B; b++)
        for (int64_t h = 0; h < H; h++)
            for (int64_t t = 0; t < T; t++) {
                int64_t base = ((t * B + b) * H + h) * D;
                int64_t ub = (t / m->tok_div) * m->sj + b * m->sb + h * m->sh;
                uint16_t r = f2h(0.0f);
                for (int64_t c = 0; c < D; c++) {
                    int64_t u = ub + c * m->sc;
                    r = chain_step(r, (int)codes[base + c] + (int)min_int[u], scale[u], q[(b * H + h) * D + c], fused);
                }
                S[(b * H + h) * T + t] = r;
            }
}

/* The fused V kernel's partial outputs (kernels.cu:350-407, 778-861): for every group g of 128 tokens,
 * C[g, b, h, c] = the fp16 chain over the group's tokens of half(code + min_int[t]) * scale[t] * P[b, h, t]. */
void orc_pv_fp16chain(const uint8_t *codes, const int16_t *min_int, const uint16_t *scale, const orc_qmeta *m,
                      int64_t T, int64_t B, int64_t H, int64_t D, const uint16_t *P, uint16_t *C, int fused) {
    for (int64_t g = 0; g < T / 128; g++)
        for (int64_t b = 0; b < B; b++)
            for (int64_t h = 0; h < H; h++)
                for (int64_t c = 0; c < D; c++) {
                    uint16_t r = f2h(0.0f);
                    for (int64_t t = g * 128; t < (g + 1) * 128; t++) {
                        int64_t u = (t / m->tok_div) * m->sj + b * m->sb + h * m->sh + c * m->sc;
                        r = chain_step(r, (int)codes[((t * B + b) * H + h) * D + c] + (int)min_int[u], scale[u],
                                       P[(b * H + h) * T + t], fused);
                    }
                    C[((g * B + b) * H + h) * D + c] = r;
                }
}

/* kernels.cu:778-861 + :350-407 (fused V) followed by the sum over token groups
 * of models/cache/kvcomp_encode.py:275:
 *     O[b, hq, c] = sum_t P[b, hq, t] * x^_V[t, b, hkv, c]. */
void orc_pv(const uint8_t *codes, const int16_t *min_int, const uint16_t *scale, const orc_qmeta *m,
            int64_t T, int64_t B, int64_t Hkv, int64_t Hq, int64_t D, const float *P, float *O) {
    int64_t G = Hq / Hkv;
#pragma omp parallel for collapse(2) schedule(static)
    for (int64_t b = 0; b < B; b++)
        for (int64_t hq = 0; hq < Hq; hq++) {
            int64_t h = hq / G;
            double acc[1024];
            for (int64_t c = 0; c < D; c++) acc[c] = 0;
            for (int64_t t = 0; t < T; t++) {
                int64_t base = ((t * B + b) * Hkv + h) * D;
                int64_t ub = (t / m->tok_div) * m->sj + b * m->sb + h * m->sh;
                double p = P[(b * Hq + hq) * T + t];
                for (int64_t c = 0; c < D; c++) {
                    int64_t u = ub + c * m->sc;
                    acc[c] += p * (double)((int)codes[base + c] + (int)min_int[u]) * (double)h2f(scale[u]);
                }
            }
            for (int64_t c = 0; c < D; c++) O[(b * Hq + hq) * D + c] = (float)acc[c];
        }
}

/* models/llama.py:211-234 (eager_attention_forward) for one decode step over the
 * dequantised cache plus an optional uncompressed fp16 tail (the recent window,
 * models/cache/kvcomp_encode.py:151):
 *     O = softmax(q K^T * scaling) V      (no mask: one query attends to all)
 * evaluated in double so that it is the exact value both fp16/fp32 pipelines
 * approximate.  ktail/vtail: [Tr, B, Hkv, D] fp16 or NULL. */
void orc_attention(const uint8_t *kc, const int16_t *kmin, const uint16_t *kscale, const orc_qmeta *km,
                   const uint8_t *vc, const int16_t *vmin, const uint16_t *vscale, const orc_qmeta *vm,
                   int64_t T, int64_t B, int64_t Hkv, int64_t Hq, int64_t D,
                   const uint16_t *ktail, const uint16_t *vtail, int64_t Tr,
                   const uint16_t *q, float scaling, float *O) {
    int64_t G = Hq / Hkv, TT = T + Tr;
#pragma omp parallel for collapse(2) schedule(dynamic)
    for (int64_t b = 0; b < B; b++)
        for (int64_t hq = 0; hq < Hq; hq++) {
            int64_t h = hq / G;
            double *s = (double *)malloc(sizeof(double) * (TT > 0 ? TT : 1));
            double mx = -INFINITY;
            for (int64_t t = 0; t < TT; t++) {
                double acc = 0;
                if (t < T) {
                    int64_t base = ((t * B + b) * Hkv + h) * D;
                    int64_t ub = (t / km->tok_div) * km->sj + b * km->sb + h * km->sh;
                    for (int64_t c = 0; c < D; c++) {
                        int64_t u = ub + c * km->sc;
                        acc += (double)((int)kc[base + c] + (int)kmin[u]) * (double)h2f(kscale[u]) *
                               (double)h2f(q[(b * Hq + hq) * D + c]);
                    }
                } else {
                    int64_t base = (((t - T) * B + b) * Hkv + h) * D;
                    for (int64_t c = 0; c < D; c++)
                        acc += (double)h2f(ktail[base + c]) * (double)h2f(q[(b * Hq + hq) * D + c]);
                }
                s[t] = acc * (double)scaling;
                if (s[t] > mx) mx = s[t];
            }
            double l = 0;
            for (int64_t t = 0; t < TT; t++) { s[t] = exp(s[t] - mx); l += s[t]; }
            double acc[1024];
            for (int64_t c = 0; c < D; c++) acc[c] = 0;
            for (int64_t t = 0; t < TT; t++) {
                double p = s[t] / l;
                if (t < T) {
                    int64_t base = ((t * B + b) * Hkv + h) * D;
                    int64_t ub = (t / vm->tok_div) * vm->sj + b * vm->sb + h * vm->sh;
                    for (int64_t c = 0; c < D; c++) {
                        int64_t u = ub + c * vm->sc;
                        acc[c] += p * (double)((int)vc[base + c] + (int)vmin[u]) * (double)h2f(vscale[u]);
                    }
                } else {
                    int64_t base = (((t - T) * B + b) * Hkv + h) * D;
                    for (int64_t c = 0; c < D; c++) acc[c] += p * (double)h2f(vtail[base + c]);
                }
            }
            for (int64_t c = 0; c < D; c++) O[(b * Hq + hq) * D + c] = (float)acc[c];
            free(s);
        }
}

/* kernels.cu:1192-1219 (k_mat_vec_mul): dense q.k over uncompressed fp16 K
 * [ctx, 1, H, 128]; the reference indexes q by (vector index % head_num), which
 * is the head of the row because rows are (token, head) in that order. */
void orc_k_matvec(const uint16_t *k, const uint16_t *q, int64_t ctx, int64_t H, int64_t D, float *out) {
    for (int64_t r = 0; r < ctx * H; r++) {
        double acc = 0;
        for (int64_t c = 0; c < D; c++) acc += (double)h2f(k[r * D + c]) * (double)h2f(q[(r % H) * D + c]);
        out[r] = (float)acc;
    }
}
