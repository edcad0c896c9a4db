"""Drop-in for the reference's `triteia_cuda` extension module.

Same callables, argument order, defaults and error behaviour as the pybind11 module built from
triteia/csrc/ops/ops.cpp (`mul_2_4` :88, `dispatch_sgmv_cutlass` :120, `dispatch_bgmv` :177,
`bmm_2_4` :240, `sbmm_forloop` :279, `sbmm_2_4` :295, registrations :350-364), implemented as a
thin shim over the C ABI of libtriteia_b200.so: shapes become integers, tensors become device
pointers, the launch goes to torch's current stream of the tensors' device.
"""
import torch

from . import _lib
from ._lib import lib, ptr, stream_of, dev_of


def _check_input(t, name):
    if not t.is_cuda:
        raise RuntimeError(f"{name} must be a CUDA tensor")
    if not t.is_contiguous():
        raise RuntimeError(f"{name} must be contiguous")


def _group_arg(num_groups, prob_k, what):
    """Dense-K group size (-1 or K / num_groups) from the leading dimension of the scales."""
    if num_groups == 1:
        return -1
    if prob_k % num_groups != 0:
        raise RuntimeError(f"k={prob_k} not compatible with {num_groups} groups.")
    return prob_k // num_groups


def _raise_shape(err, prob_m, prob_n, prob_k, thread_k, thread_m, groupsize, tname="thread_m"):
    if err == _lib.ERR_PROB_SHAPE:
        raise RuntimeError(
            f"Problem (m={prob_m}, n={prob_n}, k={prob_k}) not compatible with thread_k={thread_k}, "
            f"{tname}={thread_m}."
        )
    if err == _lib.ERR_KERN_SHAPE:
        raise RuntimeError(
            f"No kernel implementation for thread_k={thread_k}, {tname}={thread_m}, groupsize={groupsize}."
        )
    _lib.check(err, "triteia_cuda")


def mul_2_4(A, B, meta, C, s, workspace, thread_k=-1, thread_m=-1, sms=-1, max_par=8):
    for t, n in ((A, "A"), (B, "B"), (meta, "meta"), (C, "C"), (s, "s")):
        _check_input(t, n)
    prob_n, prob_m, prob_k = A.size(0), C.size(1), A.size(1)
    groupsize = _group_arg(s.size(0), prob_k, "mul_2_4")
    if workspace.numel() < prob_m // 128 * max_par:
        raise RuntimeError(f"workspace must be of size at least {prob_m // 128 * max_par}.")
    err = lib.trb_mul_2_4(ptr(A), ptr(B), ptr(meta), ptr(C), ptr(s), prob_m, prob_n, prob_k, ptr(workspace),
                          groupsize, dev_of(A), stream_of(A), thread_k, thread_m, sms, max_par)
    _raise_shape(err, prob_m, prob_n, prob_k, thread_k, thread_m, groupsize)


def bmm_2_4(A, B, meta, C, s, workspace, thread_k=-1, thread_m=-1, sms=-1, max_par=16):
    """A [n, 1, k], B [n, k/32, 2m], meta [n, m, k/16], C [n, 1, m], s [n, G, m]."""
    for t, n in ((A, "A"), (B, "B"), (meta, "meta"), (C, "C"), (s, "s")):
        _check_input(t, n)
    prob_n, prob_m, prob_k = A.size(0), C.size(2), A.size(2)
    if A.size(1) != 1:
        raise RuntimeError("bmm_2_4 takes one token per request: A must be [n, 1, k]")
    groupsize = _group_arg(s.size(1), prob_k, "bmm_2_4")
    err = lib.trb_bmm_2_4(ptr(A), ptr(B), ptr(meta), ptr(C), ptr(s), prob_m, prob_n, prob_k, ptr(workspace),
                          groupsize, dev_of(A), stream_of(A), thread_k, thread_m, sms, max_par)
    _raise_shape(err, prob_m, prob_n, prob_k, thread_k, thread_m, groupsize)


def sbmm_2_4(A, B, meta, C, s, indices, workspace, starts, counts, thread_k=-1, thread_n=-1, sms=-1, max_par=8):
    for t, n in ((A, "A"), (B, "B"), (meta, "meta"), (C, "C"), (s, "s"), (indices, "indices"),
                 (starts, "starts"), (counts, "counts")):
        _check_input(t, n)
    for t, n in ((indices, "indices"), (starts, "starts"), (counts, "counts")):
        if t.dtype != torch.int32:
            raise RuntimeError(f"{n} must be an int32 tensor")
    prob_n, prob_m, prob_k, prob_r = A.size(0), C.size(1), A.size(1), indices.size(0)
    groupsize = _group_arg(s.size(1), prob_k, "sbmm_2_4")
    err = lib.trb_sbmm_2_4(ptr(A), ptr(B), ptr(meta), ptr(C), ptr(s), ptr(indices), ptr(starts), ptr(counts),
                           prob_m, prob_n, prob_k, prob_r, ptr(workspace), groupsize, dev_of(A), stream_of(A),
                           thread_k, thread_n, sms, max_par)
    _raise_shape(err, prob_m, prob_n, prob_k, thread_k, thread_n, groupsize, "thread_n")


def sbmm_forloop(A, B, meta, C, s, indices, workspace, starts, counts, thread_k=-1, thread_n=-1, sms=-1, max_par=8):
    """One mul_2_4 per segment, two host reads per segment (as ops.cpp:279-293)."""
    for i in range(indices.size(0)):
        start = int(starts[i].item())
        end = start + int(counts[i].item())
        d = int(indices[i].item())
        mul_2_4(A[start:end], B[d], meta[d], C[start:end], s[d], workspace[i], thread_k, thread_n, sms, max_par)


def dispatch_bgmv(y, x, w, indicies, layer_idx, scale):
    for t, n in ((y, "y"), (x, "x"), (w, "w"), (indicies, "indicies")):
        _check_input(t, n)
    if y.dim() != 2 or x.dim() != 2 or w.dim() != 4 or indicies.dim() != 1:
        raise RuntimeError("dispatch_bgmv: y and x must be 2D, w 4D, indicies 1D")
    B, h_in, h_out, num_layers = x.size(0), x.size(1), y.size(1), w.size(1)
    if w.size(3) != h_in or w.size(2) != h_out or indicies.size(0) != B or y.size(0) != B:
        raise RuntimeError(f"CHECK_EQ failed: w {tuple(w.shape)} vs h_in={h_in}, h_out={h_out}, batch={B}")
    if indicies.dtype != torch.int64:
        raise RuntimeError("indicies must be an int64 tensor")
    if x.dtype not in (torch.float16, torch.bfloat16) or y.dtype != x.dtype or w.dtype != x.dtype:
        raise RuntimeError(f"No suitable kernel. h_in={h_in} h_out={h_out} dtype={x.dtype}")
    err = lib.trb_bgmv(ptr(y), ptr(x), ptr(w), ptr(indicies), B, h_in, h_out, num_layers, int(layer_idx),
                       float(scale), _lib.dtype_tag(x.dtype), dev_of(x), stream_of(x))
    if err == _lib.ERR_KERN_SHAPE:
        raise RuntimeError(f"No suitable kernel. h_in={h_in} h_out={h_out} dtype={x.dtype}")
    _lib.check(err, "dispatch_bgmv")


def sgmv_cutlass_tmp_size(num_problems):
    return int(lib.trb_sgmv_tmp_size(int(num_problems)))


def sgmv_cutlass(y, x, w_ptr, s, tmp, layer_idx):
    for t, n in ((y, "y"), (x, "x"), (w_ptr, "w_ptr"), (s, "s"), (tmp, "tmp")):
        _check_input(t, n)
    if y.dim() != 2 or x.dim() != 2 or w_ptr.dim() != 1 or s.dim() != 1 or tmp.dim() != 1:
        raise RuntimeError("sgmv_cutlass: y and x must be 2D; w_ptr, s and tmp 1D")
    num_problems = s.size(0) - 1
    if tmp.size(0) != sgmv_cutlass_tmp_size(num_problems):
        raise RuntimeError(f"CHECK_EQ(tmp.size(0), sgmv_tmp_size(num_problems)) failed. "
                           f"{tmp.size(0)} vs {sgmv_cutlass_tmp_size(num_problems)}")
    if w_ptr.dtype != torch.int64 or s.dtype != torch.int32 or w_ptr.size(0) != num_problems:
        raise RuntimeError("w_ptr must be int64 [S], s int32 [S + 1]")
    if x.dtype not in (torch.float16, torch.bfloat16) or y.dtype != x.dtype:
        raise RuntimeError(f"No suitable kernel. dtype={x.dtype}")
    err = lib.trb_sgmv(ptr(y), ptr(x), ptr(w_ptr), ptr(s), ptr(tmp), num_problems, x.size(1), y.size(1),
                       int(layer_idx), _lib.dtype_tag(x.dtype), dev_of(x), stream_of(x))
    if err == _lib.ERR_KERN_SHAPE:
        raise RuntimeError(f"No suitable kernel. dtype={x.dtype}")
    _lib.check(err, "sgmv_cutlass")


def gelu_quick(out, input):
    """out = input * sigmoid(1.702 * input) (the pybind module's gelu_quick, ops.cpp:363)."""
    _check_input(out, "out")
    _check_input(input, "input")
    if out.shape != input.shape or out.dtype != input.dtype:
        raise RuntimeError("gelu_quick: out and input must have the same shape and dtype")
    _lib.check(lib.trb_gelu_quick(ptr(out), ptr(input), input.numel(), _lib.dtype_tag(input.dtype), dev_of(input),
                                  stream_of(input)), "gelu_quick")


def silu_and_mul(out, input):
    """out[..., :d] = silu(input[..., :d]) * input[..., d:] (declared at ops.cpp:335)."""
    _check_input(out, "out")
    _check_input(input, "input")
    d = input.size(-1) // 2
    if input.size(-1) != 2 * d or out.size(-1) != d or out.numel() * 2 != input.numel():
        raise RuntimeError("silu_and_mul: input must be [..., 2 * d] and out [..., d]")
    _lib.check(lib.trb_silu_and_mul(ptr(out), ptr(input), input.numel() // (2 * d) if d else 0, d,
                                    _lib.dtype_tag(input.dtype), dev_of(input), stream_of(input)), "silu_and_mul")


def _rotary(positions, query, key, head_size, cos_sin_cache, is_neox, rot_dim, offsets):
    for t, n in ((positions, "positions"), (query, "query"), (key, "key"), (cos_sin_cache, "cos_sin_cache")):
        _check_input(t, n)
    if positions.dtype != torch.int64:
        raise RuntimeError("positions must be an int64 tensor")
    num_tokens = query.numel() // query.size(-1)
    num_heads, num_kv_heads = query.size(-1) // head_size, key.size(-1) // head_size
    _lib.check(lib.trb_rotary_embedding(ptr(positions), ptr(query), ptr(key), ptr(cos_sin_cache), ptr(offsets),
                                        num_tokens, rot_dim, query.stride(-2), key.stride(-2), num_heads, num_kv_heads,
                                        head_size, int(bool(is_neox)), _lib.dtype_tag(query.dtype), dev_of(query),
                                        stream_of(query)), "rotary_embedding")


def rotary_embedding(positions, query, key, head_size, cos_sin_cache, is_neox):
    """In place; query [..., num_heads * head_size], key [..., num_kv_heads * head_size],
    cos_sin_cache [max_position, rot_dim] (pos_encoding_kernels.cu:118-160)."""
    _rotary(positions, query, key, head_size, cos_sin_cache, is_neox, cos_sin_cache.size(1), None)


def batched_rotary_embedding(positions, query, key, head_size, cos_sin_cache, is_neox, rot_dim, cos_sin_cache_offsets):
    """rotary_embedding with a per-token row offset into the cache (pos_encoding_kernels.cu:166-213)."""
    _check_input(cos_sin_cache_offsets, "cos_sin_cache_offsets")
    if cos_sin_cache_offsets.dtype != torch.int64:
        raise RuntimeError("cos_sin_cache_offsets must be an int64 tensor")
    _rotary(positions, query, key, head_size, cos_sin_cache, is_neox, rot_dim, cos_sin_cache_offsets)
