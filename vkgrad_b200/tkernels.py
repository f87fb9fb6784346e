"""Transformer ops under the reference's names and calling conventions.

`make_transformer_kernels(dev)` returns the dictionary tkernels.py:17-389 of the
reference returns; every entry is called `TK[name](buffers, n, *push,
graph=None)` with the same buffer order and push values, so a model written
against the reference's kernels runs unchanged.  The row kernels keep the
reference's dispatch convention n = rows * dev.row_subgroup_size (one 32-lane
group per row, tkernels.py:103-104).

Differences that do not change results: column sums go through a fixed-order
two-stage reduction instead of float atomics (so `col_sum_chunk*` is
deterministic), and `col_sum_zero` is a memset.
"""

from .kernels import Elementwise, _check
from ._lib import F16, F32


def make_transformer_kernels(dev):
    lib, h = dev.lib, dev.handle
    W = dev.row_subgroup_size
    K = {}

    def op(name, nbuf, fn, prepare=None):
        K[name] = Elementwise(dev, name, fn, nbuf, prepare)

    op("layernorm", 6, lambda b, n, D: _check(
        lib.vkg_layernorm(h, b[0].dptr, b[1].dptr, b[2].dptr, b[3].dptr, b[4].dptr, b[5].dptr,
                          n // W, int(D)), "layernorm"))
    op("layernorm_bwd", 8, lambda b, n, D: _check(
        lib.vkg_layernorm_bwd(h, b[0].dptr, b[1].dptr, b[2].dptr, b[3].dptr, b[4].dptr, None,
                              b[5].dptr, None, b[6].dptr, b[7].dptr, None, None, None, None,
                              n // W, int(D)), "layernorm_bwd"))
    op("attn_softmax", 2, lambda b, n, T, scale: _check(
        lib.vkg_attn_softmax(h, b[0].dptr, None, b[1].dptr, n // W, int(T), 1, float(scale), 0),
        "attn_softmax"))
    op("attn_softmax_doc", 3, lambda b, n, T, H, scale: _check(
        lib.vkg_attn_softmax(h, b[0].dptr, b[1].dptr, b[2].dptr, n // W, int(T), int(H),
                             float(scale), 0), "attn_softmax_doc"))
    op("attn_softmax_bwd", 3, lambda b, n, T, scale: _check(
        lib.vkg_attn_softmax_bwd(h, b[0].dptr, b[1].dptr, b[2].dptr, n // W, int(T),
                                 float(scale), 0), "attn_softmax_bwd"))
    op("split_qkv", 5, lambda b, n, D, T, H, hd: _check(
        lib.vkg_split_qkv(h, b[0].dptr, b[1].dptr, b[2].dptr, b[3].dptr, b[4].dptr, n,
                          int(D), int(T), int(H), int(hd)), "split_qkv"))
    op("merge_qkv_grad", 4, lambda b, n, D, T, H, hd: _check(
        lib.vkg_merge_qkv_grad(h, b[0].dptr, b[1].dptr, b[2].dptr, b[3].dptr, n,
                               int(D), int(T), int(H), int(hd)), "merge_qkv_grad"))
    op("col_sum_zero", 1, lambda b, n: _check(
        lib.vkg_memset0(h, b[0].dptr, n * 4), "col_sum_zero"))

    def col_sum_scratch(b, n, ncol, nrow, nchunk):
        return dev.scratch(lib.vkg_col_sum_scratch_floats(int(ncol), int(nrow)) * 4)

    def col_sum_chunk(dtype):
        def go(b, n, ncol, nrow, nchunk, scratch):
            _check(lib.vkg_col_sum_det(h, b[0].dptr, dtype, b[1].dptr, scratch.dptr, int(ncol),
                                       int(nrow), 1), "col_sum_chunk")
        return go

    op("col_sum_chunk", 2, col_sum_chunk(F32), col_sum_scratch)
    op("col_sum_chunk16", 2, col_sum_chunk(F16), col_sum_scratch)
    op("merge_heads", 2, lambda b, n, D, T, H, hd: _check(
        lib.vkg_merge_heads(h, b[0].dptr, b[1].dptr, n, int(D), int(T), int(H), int(hd)),
        "merge_heads"))
    op("split_heads", 2, lambda b, n, D, T, H, hd: _check(
        lib.vkg_split_heads(h, b[0].dptr, b[1].dptr, n, int(D), int(T), int(H), int(hd)),
        "split_heads"))
    op("embed", 4, lambda b, n, D, T: _check(
        lib.vkg_embed(h, b[0].dptr, b[1].dptr, b[2].dptr, None, b[3].dptr, n, int(D), int(T)),
        "embed"))
    op("embed_bwd", 4, lambda b, n, D, T: _check(
        lib.vkg_embed_bwd(h, b[0].dptr, b[1].dptr, None, b[2].dptr, b[3].dptr, n, int(D), int(T)),
        "embed_bwd"))
    op("embed_doc", 5, lambda b, n, D, T: _check(
        lib.vkg_embed(h, b[0].dptr, b[1].dptr, b[2].dptr, b[3].dptr, b[4].dptr, n, int(D), int(T)),
        "embed_doc"))
    op("embed_doc_bwd", 5, lambda b, n, D, T: _check(
        lib.vkg_embed_bwd(h, b[0].dptr, b[1].dptr, b[2].dptr, b[3].dptr, b[4].dptr, n, int(D),
                          int(T)), "embed_doc_bwd"))
    op("residual", 4, lambda b, n, D: _check(
        lib.vkg_residual(h, b[0].dptr, b[1].dptr, b[2].dptr, b[3].dptr, n, int(D)), "residual"))
    op("add", 3, lambda b, n: _check(
        lib.vkg_add(h, b[0].dptr, b[1].dptr, b[2].dptr, None, n), "add"))
    op("add_bias", 2, lambda b, n, ncol: _check(
        lib.vkg_add_bias(h, b[0].dptr, b[1].dptr, n, int(ncol)), "add_bias"))
    op("to16", 2, lambda b, n: _check(
        lib.vkg_cast16(h, b[0].dptr, b[1].dptr, n), "to16"))
    return K
