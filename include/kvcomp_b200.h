/*
 * kvcomp_b200 -- C ABI of the B200 (sm_100a) KV-cache compression hot path.
 *
 * Drop-in boundary for the operator module `kvcomp_cuda` of BoJiang03/kvcomp
 * (kvcomp_cuda_extension/export_kvcomp.cpp:8-24, prototypes include/kernels.h:56-133,
 * include/huffman.h:26) and for the torch-side quantiser its cache class calls
 * (utils/compute.py:93-106).  Plain pointers and sizes only: every pointer named
 * "device" is a CUDA device pointer of the current device, every entry point takes the
 * stream to launch on, nothing here allocates device memory, synchronises the device or
 * changes the current device, and nothing aborts: every entry point returns a KVC_* code
 * and kvc_last_error() gives the text.
 *
 * Tensors use the reference's CUDA-path layout: token-major [T, B, H, 128] (T tokens,
 * B sequences, H KV heads, head_dim 128 = one Huffman vector); `cols` = B*H.
 *
 * Compressed stream format (kernels.cu:181-235,419-596; include/kernels.h:25-32), kept
 * bit for bit:
 *   vector  = 128 symbols, codes concatenated MSB first, zero padded to a whole byte
 *             K: the 128 channels of (token, col)        V: 128 tokens of one channel column
 *   block   = 64 vectors back to back
 *             K: tokens 64j..64j+63 of one col, id = j*cols + col
 *             V: token group g (128 tokens) x 64 channel columns, id = g*cols*2 + m
 *   thread_info[block*64+v] (u16) = (end byte of v inside the block << 3) | pad bits
 *   block_info[block]       (8 B) = { u32 byte offset in the stream, u16 byte count, 2 B zero }
 * Blocks of one encode call are laid out in ascending id (the reference's order depends on
 * an atomic cursor; every order is a valid stream).
 */
#ifndef KVCOMP_B200_H
#define KVCOMP_B200_H

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define KVC_VERSION 1

/* return codes */
#define KVC_OK            0
#define KVC_ERR_ARG       1   /* null pointer, bad shape, unsupported size or mode */
#define KVC_ERR_CUDA      2   /* a CUDA runtime call failed; text in kvc_last_error() */
#define KVC_ERR_CAPACITY  3   /* a caller-provided buffer is too small */

/* bits of the device status word (int32, OR-ed by kernels, never cleared by them).  The
 * reference ignores every one of these conditions (include/utils.h:7-15 aborts on host
 * asserts only); here they are reported and the call still completes. */
#define KVC_FLAG_ZERO_SCALE      0x001  /* quantiser: a unit is constant (reference: NaN codes) */
#define KVC_FLAG_MIN_OVERFLOW    0x002  /* quantiser: min_int does not fit the requested width */
#define KVC_FLAG_CODE_OVERFLOW   0x004  /* quantiser: a code is outside 0..255 */
#define KVC_FLAG_SYMBOL_MISSING  0x008  /* encoder: symbol without a code was dropped */
#define KVC_FLAG_VECTOR_LONG     0x010  /* encoder: a vector exceeds the reference's scratch (K 128 B, V 256 B) */
#define KVC_FLAG_BLOCK_LONG      0x020  /* encoder: a block exceeds 8191 B, its u16 fields are invalid */
#define KVC_FLAG_STREAM_FULL     0x040  /* encoder: `encoded` capacity exceeded, output truncated */
#define KVC_FLAG_BAD_STREAM      0x080  /* decoder: a vector did not decode to 128 symbols */
#define KVC_FLAG_CODE_TOO_LONG   0x100  /* codebook: a code is longer than 32 bits */
#define KVC_FLAG_NO_SYMBOLS      0x200  /* codebook: empty histogram */
#define KVC_FLAG_WAIT_TIMEOUT    0x400  /* a bounded device-side wait gave up */

typedef void *kvc_stream_t;   /* a cudaStream_t; NULL = the legacy default stream */

/* quantisation modes (utils/compute.py:5-10) */
#define KVC_MODE_BLOCK   0
#define KVC_MODE_CHANNEL 1
#define KVC_MODE_TOKEN   2
#define KVC_MODE_VECTOR  3

/* Where the (min_int, scale) of element (t, b, h, c) live:
 *     unit = (t / tok_div) * sj + b * sb + h * sh + c * sc
 * A stride of 0 means the unit spans that dimension.  kvc_qmeta_make() fills it for the
 * reference's unit shapes. */
typedef struct {
    const void *min_int;   /* device, int8 (reference, kvcomp_encode.py:97) or int16 */
    const void *scale;     /* device, fp16 */
    int32_t min_bytes;     /* 1 or 2 */
    int32_t tok_div;
    int64_t sj, sb, sh, sc;
} kvc_qmeta;

/* One compressed K or V cache of T tokens (all store calls so far). */
typedef struct {
    const uint8_t *encoded;       /* device; readable up to the next 16-byte boundary past its end */
    int64_t encoded_bytes;
    const void *block_info;       /* device, 8-byte records */
    const uint16_t *thread_info;  /* device */
    const void *book;             /* device, KVC_BOOK_BYTES, from kvc_build_codebook / kvc_book_from_tree */
    kvc_qmeta q;
    int32_t max_block_bytes;      /* upper bound of any block's byte count (kvc_encode reports it); 0 = unknown
                                     (8191 is assumed).  A tight bound lets more CTAs share an SM. */
    int32_t reserved;
} kvc_cache;

/* ---- codebook object (device blob) ------------------------------------------------ */
#define KVC_LUT_BITS        12
#define KVC_BOOK_OFF_ENC    64                       /* 256 x {u32 code, u32 length}, symbol-indexed */
#define KVC_BOOK_OFF_REFTREE (KVC_BOOK_OFF_ENC + 2048)   /* 512 x 3-byte nodes, reference format */
#define KVC_BOOK_OFF_TREE   (KVC_BOOK_OFF_REFTREE + 1536) /* 512 x u32 wide nodes */
#define KVC_BOOK_OFF_LUT    (KVC_BOOK_OFF_TREE + 2048)    /* (1<<KVC_LUT_BITS) x u32 decode-table entries */
#define KVC_BOOK_BYTES      (KVC_BOOK_OFF_LUT + 4 * (1 << KVC_LUT_BITS))

typedef struct {             /* first 32 bytes of the blob */
    int32_t n_symbols;       /* distinct symbols */
    int32_t min_sym, max_sym;
    int32_t max_len;         /* longest code in bits */
    int32_t n_nodes;         /* nodes of the reference-format decode tree */
    int32_t flags;           /* KVC_FLAG_* raised while building */
    int32_t lut_bits;
    int32_t escape;          /* 1: some decode-table entry holds no complete code (a code longer than the
                              * window, or bit patterns that belong to no code): decoders test for it */
} kvc_book_header;

const char *kvc_last_error(void);
int kvc_version(void);

/* calculate_buffer_size (kernels.cu:893-917): out = {block_info bytes, thread_info bytes,
 * 8 (the reference's cursor, unused here), numel (encoded capacity the reference allocates)}.
 * tokens = T of the call, hidden = B*H*128. */
int kvc_buffer_sizes(int64_t tokens, int64_t hidden, int is_k, int64_t out[4]);

/* Fill q->{tok_div,sj,sb,sh,sc} for a mode.  batch_shared = 1: units span the batch
 * (the CUDA path's tables, models/cache/kvcomp_encode.py:10-13); 0: per sequence
 * (utils/compute.py:138-143).  Returns the number of units in *n_units. */
int kvc_qmeta_make(int mode, int batch_shared, int64_t T, int64_t B, int64_t H, int64_t D,
                   int64_t block, kvc_qmeta *q, int64_t *n_units);

/* quant (utils/compute.py:93-106; src/compute.cpp:40-58) fused with the uint8/int8
 * narrowing of models/cache/kvcomp_encode.py:97-98.  x: device fp16 [T,B,H,D], D % 8 == 0.
 * codes: device u8 [T,B,H,D]; min_int (min_bytes 1|2) and scale (fp16): one per unit in
 * the order kvc_qmeta_make describes.  hist (optional, device u64[256]) accumulates the
 * code histogram of this call.  workspace: KVC_MODE_BLOCK needs 8 bytes per unit
 * (kvc_quantize_workspace), others none.  status: device int32, OR-ed. */
int64_t kvc_quantize_workspace(int mode, int batch_shared, int64_t T, int64_t B, int64_t block);
int kvc_quantize(const void *x, int64_t T, int64_t B, int64_t H, int64_t D,
                 int mode, int batch_shared, int64_t block, float rel,
                 uint8_t *codes, void *min_int, int min_bytes, void *scale,
                 unsigned long long *hist, void *workspace, int64_t workspace_bytes,
                 int32_t *status, kvc_stream_t stream);

/* The quantiser in two calls, for caches whose KV heads are split over several GPUs.  BlockQuant and
 * TokenQuant units span the heads (models/cache/kvcomp_encode.py:10-13, utils/compute.py:138-143), so a
 * rank that holds some of the heads cannot derive scale and min_int alone.  kvc_quant_minmax writes the
 * extremes of this rank's x per unit (device fp16 mn_out[units], mx_out[units], units as in
 * kvc_qmeta_make); the ranks take the elementwise minimum / maximum over all of them; kvc_quantize_ranged
 * then quantises x with the given extremes.  One rank holding every head gets the bits of kvc_quantize.
 * Other modes are refused: their units are local to a head.  workspace: 8 bytes per unit. */
int kvc_quant_minmax(const void *x, int64_t T, int64_t B, int64_t H, int64_t D, int mode, int batch_shared,
                     int64_t block, void *mn_out, void *mx_out, void *workspace, int64_t workspace_bytes,
                     kvc_stream_t stream);
int kvc_quantize_ranged(const void *x, int64_t T, int64_t B, int64_t H, int64_t D, int mode, int batch_shared,
                        int64_t block, float rel, const void *mn_in, const void *mx_in,
                        uint8_t *codes, void *min_int, int min_bytes, void *scale, unsigned long long *hist,
                        void *workspace, int64_t workspace_bytes, int32_t *status, kvc_stream_t stream);

/* The rotary embedding the cache applies to new keys (models/cache/kvcomp_quant.py:43-48 with
 * utils/compute.py:25-33: t * cos + rotate_half(t) * sin, each op rounded to fp16) fused with the
 * transposition into the cache's token-major layout: x device fp16 [B, H, t, D] (as the attention layer
 * hands it over) -> out device fp16 [t, B, H, D].  cos / sin: device fp16 [B, t, D], or [1, t, D] with
 * cos_batch_stride = 0.  Same bits as the torch ops.  cos_ = sin_ = NULL: no rotation, the transposition
 * alone (how new values reach the token-major recent window).  out may be a row range of a larger buffer. */
int kvc_rope_store(const void *x, const void *cos_, const void *sin_, void *out, int64_t B, int64_t H, int64_t t,
                   int64_t D, int64_t cos_batch_stride, kvc_stream_t stream);
/* kvc_rope_store for the new keys (rotated) and for the new values (not rotated) of a decode step in one
 * launch: k, v device fp16 [B, H, t, D] -> kout, vout device fp16 [t, B, H, D]. */
int kvc_kv_store(const void *k, const void *v, const void *cos_, const void *sin_, void *kout, void *vout,
                 int64_t B, int64_t H, int64_t t, int64_t D, int64_t cos_batch_stride, kvc_stream_t stream);

/* (codes + min_int) * scale -> fp16 (models/cache/kvcomp_encode.py:146). */
int kvc_dequant(const uint8_t *codes, const kvc_qmeta *q, int64_t T, int64_t B, int64_t H, int64_t D,
                void *out, kvc_stream_t stream);

/* torch::bincount of build_codebook (src/huffman.cpp:105-109): hist[256] += counts. */
int kvc_histogram(const uint8_t *codes, int64_t n, unsigned long long *hist, kvc_stream_t stream);

/* gen_huffman_codes + build_encode_code_book + build_decode_code_book
 * (src/huffman.cpp:34-96,166-187,229-252) on the device, bit-identical code assignment
 * (heap tie-breaking included), plus the multi-symbol decode table the kernels use.
 * hist: device u64[256].  book: device, KVC_BOOK_BYTES, 16-byte aligned. */
int kvc_build_codebook(const unsigned long long *hist, void *book, kvc_stream_t stream);

/* Rebuild a book from a reference-format decode tensor (3-byte nodes, up to 255 nodes)
 * so that streams can be decoded by callers that only hold that tensor
 * (k_entropy_decode_cuda_export's decode_code_book argument). */
int kvc_book_from_tree(const uint8_t *ref_tree, int64_t tree_bytes, void *book, kvc_stream_t stream);

/* k_/v_entropy_encode_cuda_export (kernels.cu:919-1011).  codes: device u8 [T, cols, 128].
 * enc_table: device {u32 code,u32 length} x n_entries indexed by symbol (the reference's
 * encode tensor, or book + KVC_BOOK_OFF_ENC with 256 entries).  block_info / thread_info:
 * this call's records (the caller offsets them for later store calls).  encoded: where
 * this call's bytes go; base_offset is added to the recorded block offsets
 * (kernels.cu:476).  total_bytes: device u64[2]; [0] receives the byte count of this call,
 * [1] is raised to the largest block byte count seen (zero it to start a new maximum).
 * workspace: kvc_encode_workspace() bytes. */
int64_t kvc_encode_workspace(int64_t T, int64_t cols, int is_k);
int kvc_encode(const uint8_t *codes, int64_t T, int64_t cols, int is_k,
               const void *enc_table, int n_entries, uint32_t base_offset,
               void *block_info, uint16_t *thread_info, uint8_t *encoded, int64_t encoded_capacity,
               unsigned long long *total_bytes, void *workspace, int64_t workspace_bytes,
               int32_t *status, kvc_stream_t stream);

/* Diagnostics, no counterpart in the reference.  The encoder's CTAs learn their block's byte offset from
 * the blocks before them and wait for each at most `wait_limit` polls (0 = the default of 2^21); a wait
 * that runs out raises KVC_FLAG_WAIT_TIMEOUT, the block and every later one write nothing, and the call
 * returns.  starve != 0 makes the first block keep its byte count to itself, so that a test can see the
 * waits run out; the stream of such a call is undefined.  Process-wide, read at every launch. */
void kvc_encode_debug(int wait_limit, int starve);

/* k_/v_entropy_decode_cuda_export (kernels.cu:1013-1087): stream -> u8 codes [T, cols, 128].
 * block_info offsets are relative to `encoded`. */
int kvc_decode(const uint8_t *encoded, int64_t encoded_bytes, const void *block_info,
               const uint16_t *thread_info, const void *book, int64_t T, int64_t cols, int is_k,
               uint8_t *codes, int32_t *status, kvc_stream_t stream);
/* kvc_decode with the stream's largest block size (kvc_encode's total_bytes[1]; 0 = unknown, the
 * format's 8191): smaller staging slots let more CTAs share an SM.  A block beyond the bound is
 * skipped and flagged KVC_FLAG_BAD_STREAM. */
int kvc_decode_bounded(const uint8_t *encoded, int64_t encoded_bytes, const void *block_info,
                       const uint16_t *thread_info, const void *book, int64_t T, int64_t cols, int is_k,
                       uint32_t max_block_bytes, uint8_t *codes, int32_t *status, kvc_stream_t stream);

/* k_decode_and_mat_vec_mul_cuda_export (kernels.cu:1093-1136): raw scores
 * S[b,hq,t] = sum_c x^K[t,b,hkv,c] * q[b,hq,c], fp32 accumulation.  q: device fp16
 * [B,Hq,128]; out: device [B,Hq,T], fp16 (out_f32 = 0, the reference's C) or fp32. */
int kvc_fused_qk(const kvc_cache *k, int64_t T, int64_t B, int64_t Hkv, int64_t Hq,
                 const void *q, void *out, int out_f32, int32_t *status, kvc_stream_t stream);

/* v_decode_and_mat_vec_mul_cuda_export (kernels.cu:1138-1180): per 128-token group
 * partial[g,b,hq,c] = sum_{t in g} P[b,hq,t] * x^V[t,b,hkv,c].  P: device fp16 [B,Hq,T];
 * out: device fp16 [T/128, B, Hq, 128] (the reference's C; its caller sums over g). */
int kvc_fused_pv(const kvc_cache *v, int64_t T, int64_t B, int64_t Hkv, int64_t Hq,
                 const void *P, void *out, int32_t *status, kvc_stream_t stream);

/* One decode step of eager_attention_forward (models/llama.py:211-234) straight from the
 * compressed caches: out[b,hq,:] = softmax(q K^T * scaling) V over T compressed tokens
 * plus Tr uncompressed tail tokens (the recent window, ktail/vtail device fp16
 * [Tr,B,Hkv,128], may be NULL with Tr = 0; with T = 0 only the tail is read and k, v may
 * be NULL).  q: device fp16 [B,Hq,128]; out: device fp16
 * [B,Hq,128].  Scores never leave the SM; no fp16 K/V is written to memory.
 * Work is cut into items, one (sequence, KV head) column x one of `splits` equal runs of
 * 256-token tiles; as many CTAs as the device holds at once take items until none is left,
 * and a second small kernel merges the `splits` partial results of every head and adds the
 * tail's tokens (it does the whole step when T = 0).  splits = 0
 * picks kvc_attn_splits(T, B, Hkv, 0).  workspace: kvc_attn_workspace(B, Hq, splits) bytes
 * of device memory whose first 256 bytes the caller zeroes once before the first use (the
 * kernel leaves them zeroed); NULL is allowed when splits = 1 (a tail then costs more: the
 * first kernel reads it itself, a column's CTA at a time).  Launches that share a
 * workspace must not overlap on the device. */
int64_t kvc_attn_workspace(int64_t B, int64_t Hq, int splits);
int kvc_attn_splits(int64_t T, int64_t B, int64_t Hkv, int sm_count);
int kvc_attn_decode(const kvc_cache *k, const kvc_cache *v, int64_t T, int64_t B, int64_t Hkv, int64_t Hq,
                    const void *q, float scaling, const void *ktail, const void *vtail, int64_t Tr,
                    void *out, int splits, void *workspace, int64_t workspace_bytes,
                    int32_t *status, kvc_stream_t stream);

/* Diagnostics, no counterpart in the reference (its kernels have no device-side waits).  The attention
 * kernel waits for its staged blocks at most `wait_limit` tries (0 = the default of 2^22); a wait that
 * runs out raises KVC_FLAG_WAIT_TIMEOUT, the CTA stops taking work and the call returns.  starve != 0
 * makes the kernel announce staging bytes that it never copies, so that a test can see a wait run out
 * with nothing in flight; outputs of such a call are undefined.  Process-wide, read at every launch. */
void kvc_attn_debug(int wait_limit, int starve);

/* No counterpart in the reference.  kvc_attn_decode for callers that cannot allocate device memory
 * (a serving process whose memory pool owns the whole device, a plugin under a fixed memory budget):
 * the split-KV scratch is a fixed array inside the library (kvc_attn_static_capacity() bytes, 4 MiB,
 * held by every GPU that loads the library until the process exits) instead of a caller workspace.
 * Inputs and outputs are still the caller's.  Nothing is allocated or freed by this call.
 *  - B, Hq and splits whose scratch (kvc_attn_workspace) exceeds the capacity: KVC_ERR_CAPACITY.
 *  - The first call on a device looks the array's device address up (with that device current);
 *    make that first call outside any stream capture.
 *  - All calls on a device share the array: the counters are cleared on `stream` at the start of
 *    every call, and two calls that overlap on the GPU (different streams) race.  Calls on one
 *    stream are ordered and safe. */
int64_t kvc_attn_static_capacity(void);
int kvc_attn_decode_static(const kvc_cache *k, const kvc_cache *v, int64_t T, int64_t B, int64_t Hkv, int64_t Hq,
                           const void *q, float scaling, const void *ktail, const void *vtail, int64_t Tr,
                           void *out, int splits, int32_t *status, kvc_stream_t stream);

/* k_mat_vec_mul_cuda_export (kernels.cu:1192-1273): dense q.k over uncompressed fp16 K
 * [ctx,1,H,128], q [1,H,128] -> out fp16 [ctx,1,H].  Comparison baseline only. */
int kvc_k_matvec(const void *k, const void *q, void *out, int64_t ctx, int64_t H, kvc_stream_t stream);

#ifdef __cplusplus
}
#endif
#endif /* KVCOMP_B200_H */
