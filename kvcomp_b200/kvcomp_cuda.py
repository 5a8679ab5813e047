"""Drop-in for the reference's operator module `kvcomp_cuda`
(kvcomp_cuda_extension/export_kvcomp.cpp:8-24, stub kvcomp_cuda_extension/kvcomp_cuda.pyi:1-83).

Same names, argument order and meaning; every function forwards to libkvcomp_b200.so.  Use it as

    import kvcomp_b200.kvcomp_cuda as kvcomp_cuda          # or: sys.modules["kvcomp_cuda"] = ...

Differences a caller can observe:
  * errors raise KvcError instead of aborting the process (include/utils.h:7-15);
  * blocks of one encode call are laid out in ascending block id (the reference's order depends on
    an atomic cursor); every order is a valid stream for the reference's decoders and for these;
  * fused kernels accumulate in fp32 (block fixed-point weights, exact integer products) instead of
    fp16, take any batch size and any K/V head grouping, and work for every codebook size;
  * like the reference, every call returns only after the device finished its work.
"""
import torch

from . import ops
from ._lib import KvcError

# module attributes of the reference (export_kvcomp.cpp:9-12) and of its stub (kvcomp_cuda.pyi:8-12,
# values from kvcomp_cuda_extension/scripts/kv_com_ctx.py:7-15)
K_VEC_LEN = 128
K_VEC_PER_BLK = 64
V_VEC_LEN = 128
V_VEC_PER_BLK = 64
BLOCK_SIZE = 64
K_BUFFER_SIZE = 0
V_BUFFER_SIZE = 0
K_QUANT_DIMS = [1, 2, 3, 4]
V_QUANT_DIMS = [2, 3, 4]


def _five_d(t, name):
    if t.dim() != 5:
        raise KvcError("%s must be [nblk, blk, B, H, D]" % name)
    return t


def _timed(fn):
    """Run fn() between two CUDA events on the current stream; returns elapsed ms (the reference
    returns cudaEventElapsedTime, kernels.cu:1026-1048)."""
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    start.record()
    fn()
    stop.record()
    stop.synchronize()
    return start.elapsed_time(stop)


def calculate_buffer_size(input, is_k, head_num, head_dim):
    """kernels.cu:893-917 -> (block_infos bytes, thread_infos bytes, 8, numel)."""
    _five_d(input, "input")
    tokens = input.shape[0] * input.shape[1]
    hidden = input.shape[2] * input.shape[3] * input.shape[4]
    return ops.buffer_sizes(tokens, hidden, bool(is_k))


def build_codebook(input_tensors):
    """src/huffman.cpp:99-157 -> (shift, encode tensor, decode tensor), both CPU uint8 tensors in the
    reference's formats.  Histogram and code assignment run on the device of the inputs."""
    if not input_tensors:
        raise KvcError("build_codebook needs at least one tensor")
    dev = input_tensors[0].device
    hist = None
    for t in input_tensors:
        if t.device != dev:
            raise KvcError("All input tensors must be on the same device.")
        if t.dtype != torch.uint8:
            raise KvcError("Input tensors must be of type uint8.")
        hist = ops.histogram(t.contiguous().view(-1), hist)
    book = ops.build_codebook(hist)
    hd = book.header()
    if hd["flags"]:
        raise KvcError("build_codebook: %s" % "|".join(ops._lib.flag_names(hd["flags"])))
    shift, enc = book.ref_encode_tensor()
    return shift, enc, book.ref_decode_tensor()


def _encode(is_k, input, encode_code_book, block_infos, thread_infos, idx_offset, encoded_data,
            base_global_offset, head_num, head_dim):
    _five_d(input, "input")
    if head_dim != 128 or input.shape[4] != 128:
        raise KvcError("head_dim must be equal to K_VEC_LEN")
    tokens = input.shape[0] * input.shape[1]
    cols = input.shape[2] * input.shape[3]
    bsz, tsz, _, _ = ops.buffer_sizes(tokens, cols * 128, is_k)
    codes = input.contiguous().view(tokens, input.shape[2], input.shape[3], 128)
    total, status = ops.encode(codes, is_k, encode_code_book, block_infos, thread_infos, encoded_data,
                               base_offset=int(base_global_offset))
    n = int(total[0].item())                       # synchronises, like the reference's cudaDeviceSynchronize
    ops.read_status(status, what="entropy_encode")
    if idx_offset is not None and idx_offset.numel() >= 8:     # the reference's cursor: {blocks, bytes}
        idx_offset.view(torch.int32)[:2] = torch.tensor([bsz // 8, n], dtype=torch.int32, device=idx_offset.device)
    return encoded_data[:n], block_infos.view(torch.uint8)[:bsz], thread_infos.view(torch.uint8)[:tsz]


def k_entropy_encode_cuda_export(input, encode_code_book, block_infos, thread_infos, idx_offset, encoded_data,
                                 base_global_offset, head_num, head_dim):
    """kernels.cu:919-966.  Returns views (encoded[:n], block_infos, thread_infos) into the caller's buffers."""
    return _encode(True, input, encode_code_book, block_infos, thread_infos, idx_offset, encoded_data,
                   base_global_offset, head_num, head_dim)


def v_entropy_encode_cuda_export(input, encode_code_book, block_infos, thread_infos, idx_offset, encoded_data,
                                 base_global_offset, head_num, head_dim):
    """kernels.cu:968-1011."""
    return _encode(False, input, encode_code_book, block_infos, thread_infos, idx_offset, encoded_data,
                   base_global_offset, head_num, head_dim)


def _decode(is_k, in_tensor, block_infos, thread_infos, decode_code_book, out, head_num, head_dim):
    _five_d(out, "out")
    tokens = out.shape[0] * out.shape[1]
    book = ops.book_from_tree(decode_code_book)
    status = ops.new_status(out.device)
    codes = out.view(tokens, out.shape[2], out.shape[3], out.shape[4])
    ms = _timed(lambda: ops.decode(in_tensor, block_infos, thread_infos, book, tokens, out.shape[2], out.shape[3],
                                   is_k, out=codes, status=status))
    ops.read_status(status, what="entropy_decode")
    return ms


def k_entropy_decode_cuda_export(in_tensor, block_infos, thread_infos, decode_code_book, out, head_num, head_dim):
    """kernels.cu:1013-1049: writes uint8 codes into `out` [nblk, blk, B, H, D]; returns elapsed ms."""
    return _decode(True, in_tensor, block_infos, thread_infos, decode_code_book, out, head_num, head_dim)


def v_entropy_decode_cuda_export(in_tensor, block_infos, thread_infos, decode_code_book, out, head_num, head_dim):
    """kernels.cu:1051-1087."""
    return _decode(False, in_tensor, block_infos, thread_infos, decode_code_book, out, head_num, head_dim)


def _ref_spec(is_k, n_units, tokens, B, H):
    """Unit layout of the reference's CUDA path (models/cache/kvcomp_encode.py:10-13): one (min_int,
    scale) per 64-token block for K, per token for V; per sequence when the arrays are B times longer."""
    mode = ops.MODE_BLOCK if is_k else ops.MODE_TOKEN
    per = tokens // 64 if is_k else tokens
    if n_units == per:
        return ops.qspec(mode, True, B, H, 128, 64)
    if n_units == per * B:
        return ops.qspec(mode, False, B, H, 128, 64)
    raise KvcError("quant_min_ints has %d entries; expected %d (or %d per sequence)" % (n_units, per, per * B))


def k_decode_and_mat_vec_mul_cuda_export(decode_code_book, block_infos, thread_infos, encoded_data, quant_min_ints,
                                         quant_scales, B, C, head_num, head_dim):
    """kernels.cu:1093-1136: C[b, h, t] = sum_c (code + min_int) * scale * B[b, h, c]; returns elapsed ms.
    B: fp16 [batch, heads, 128]; C: fp16 (or fp32) [batch, heads, ctx]."""
    if B.dim() != 3 or C.dim() != 3:
        raise KvcError("B must be [batch, heads, 128] and C [batch, heads, ctx]")
    batch, hq, ctx = C.shape
    book = ops.book_from_tree(decode_code_book)
    mi = quant_min_ints.contiguous().view(-1)
    sc = quant_scales.contiguous().view(-1)
    spec = _ref_spec(True, mi.numel(), ctx, batch, head_num)
    cache = ops.make_cache(encoded_data, block_infos, thread_infos, book, mi, sc, spec)
    status = ops.new_status(C.device)
    ms = _timed(lambda: ops.fused_qk(cache, ctx, batch, head_num, B, out=C, status=status))
    ops.read_status(status, what="k_decode_and_mat_vec_mul")
    return ms


def v_decode_and_mat_vec_mul_cuda_export(decode_code_book, block_infos, thread_infos, encoded_data, quant_min_ints,
                                         quant_scales, B, C, head_num, head_dim):
    """kernels.cu:1138-1180: C[g, b, h, c] = sum over the 128 tokens of group g of
    (code + min_int) * scale * B[b, h, t]; the caller sums over g (kvcomp_encode.py:275).
    B: fp16 [batch, heads, ctx]; C: fp16 [ctx/128, batch, heads, 128]."""
    if B.dim() != 3 or C.dim() != 4:
        raise KvcError("B must be [batch, heads, ctx] and C [ctx/128, batch, heads, 128]")
    batch, hq, ctx = B.shape
    book = ops.book_from_tree(decode_code_book)
    mi = quant_min_ints.contiguous().view(-1)
    sc = quant_scales.contiguous().view(-1)
    spec = _ref_spec(False, mi.numel(), ctx, batch, head_num)
    cache = ops.make_cache(encoded_data, block_infos, thread_infos, book, mi, sc, spec)
    status = ops.new_status(C.device)
    ms = _timed(lambda: ops.fused_pv(cache, ctx, batch, head_num, B, out=C, status=status))
    ops.read_status(status, what="v_decode_and_mat_vec_mul")
    return ms


def k_mat_vec_mul_cuda_export(k, q, out):
    """kernels.cu:1221-1273: dense fp16 q.k baseline, k [ctx,1,H,128], q [1,H,128], out [ctx,1,H]."""
    if k.dim() != 4 or q.dim() != 3 or out.dim() != 3:
        raise KvcError("k must be [ctx,1,H,128], q [1,H,128], out [ctx,1,H]")
    if k.shape[1] != 1:
        raise KvcError("Batch size must be 1 for now")
    if q.shape[0] != k.shape[1] or q.shape[1] != k.shape[2] or q.shape[2] != k.shape[3]:
        raise KvcError("Head num / head dim of A and B must be equal")
    if out.shape[0] != k.shape[0] or out.shape[2] != k.shape[2]:
        raise KvcError("Context length / head num of A and C must be equal")
    return _timed(lambda: ops.k_matvec(k, q, out))
