"""ctypes binding of libshard_b200.so (the C ABI declared in include/shard_b200.h).

There is no CPU implementation behind these calls: if the library has not
been built, or a call is made without a CUDA device, the error is raised to
the caller.
"""
from __future__ import annotations

import ctypes as C
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "libshard_b200.so")

PART_STRIDE = 132
HEAD_DIM = 128


class ShardSeq(C.Structure):
    """Mirror of `struct ShardSeq` (device pointers of one layer of one sequence)."""
    _fields_ = [(name, C.c_void_p) for name in (
        "k_coeffs", "k_wprep", "v_indices", "v_centroids", "v_ch",
        "sink_k", "sink_v", "win_k", "win_v",
        "st_k_idx", "st_v_idx", "st_k_norm", "st_v_norm",
        "signs", "phase", "q", "out", "new_k", "new_v", "dec_k", "dec_v")]


class ShardDecodeShape(C.Structure):
    """Mirror of `struct ShardDecodeShape`."""
    _fields_ = [(name, C.c_int32) for name in (
        "n_q", "nkv", "rank", "n_comp", "tok_begin", "tok_end",
        "n_sink", "n_win", "n_stream", "pos_q", "partial_out", "append", "n_dec", "no_overlap", "dec_cap")]


_SIGNATURES = {
    "shard_b200_abi_version": (C.c_int, []),
    "shard_b200_status_string": (C.c_char_p, [C.c_int]),
    "shard_b200_phase_table_bytes": (C.c_size_t, [C.c_int32]),
    "shard_b200_phase_table": (C.c_int, [C.c_int32, C.c_int32, C.c_int32, C.c_void_p, C.c_void_p, C.c_void_p]),
    "shard_b200_wprep_bytes": (C.c_size_t, [C.c_int32, C.c_int32]),
    "shard_b200_decode_prepare": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_int32, C.c_int32,
                                            C.c_void_p, C.c_void_p]),
    "shard_b200_decode_workspace_bytes": (C.c_size_t, [C.POINTER(ShardDecodeShape), C.c_int32]),
    "shard_b200_decode_attn": (C.c_int, [C.c_void_p, C.c_int32, C.POINTER(ShardDecodeShape), C.c_void_p,
                                         C.c_void_p, C.c_void_p, C.c_size_t, C.c_void_p]),
    "shard_b200_decode_attn_noalloc": (C.c_int, [C.c_void_p, C.POINTER(ShardDecodeShape), C.c_void_p, C.c_void_p,
                                                 C.c_void_p]),
    "shard_b200_lse_merge": (C.c_int, [C.c_void_p, C.c_int32, C.c_int32, C.c_void_p, C.c_void_p]),
    "shard_b200_vq_assign_accumulate": (C.c_int, [C.c_void_p, C.c_void_p, C.c_int64, C.c_void_p, C.c_void_p, C.c_void_p,
                                                  C.c_void_p]),
    "shard_b200_peer_buffer_bytes": (C.c_size_t, [C.c_int32, C.c_int32]),
    "shard_b200_peer_alloc": (C.c_int, [C.c_size_t, C.c_void_p, C.c_void_p]),
    "shard_b200_peer_open": (C.c_int, [C.c_void_p, C.c_void_p]),
    "shard_b200_peer_close": (C.c_int, [C.c_void_p]),
    "shard_b200_peer_free": (C.c_int, [C.c_void_p]),
    "shard_b200_seqsplit_merge": (C.c_int, [C.c_void_p, C.c_void_p, C.c_int32, C.c_int32, C.c_int32, C.c_uint32,
                                            C.c_void_p, C.c_void_p, C.c_uint32, C.c_void_p]),
    "shard_b200_decode_attn_seqsplit": (C.c_int, [C.c_void_p, C.POINTER(ShardDecodeShape), C.c_void_p, C.c_void_p,
                                                  C.c_void_p, C.c_size_t, C.c_void_p, C.c_int32, C.c_int32,
                                                  C.c_uint32, C.c_void_p, C.c_void_p, C.c_uint32, C.c_void_p]),
    "shard_b200_seqsplit_wait_merge": (C.c_int, [C.c_void_p, C.c_int32, C.c_int32, C.c_int32, C.c_uint32,
                                                 C.c_void_p, C.c_void_p, C.c_uint32, C.c_void_p]),
    "shard_b200_decode_status": (C.c_int, [C.c_void_p, C.POINTER(C.c_int32), C.c_void_p]),
    "shard_b200_stream_quantize": (C.c_int, [C.c_void_p, C.c_int32, C.c_int32, C.c_int32, C.c_void_p,
                                             C.c_void_p]),
    "shard_b200_stream_dequant": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_int32,
                                            C.c_int32, C.c_void_p, C.c_void_p]),
    "shard_b200_undo_rope": (C.c_int, [C.c_void_p, C.c_int64, C.c_int64, C.c_int32, C.c_int32, C.c_int32,
                                       C.c_void_p, C.c_void_p, C.c_void_p]),
    "shard_b200_k_project_workspace_bytes": (C.c_size_t, [C.c_int32, C.c_int32]),
    "shard_b200_k_project": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_int32, C.c_int32, C.c_int32,
                                       C.c_void_p, C.c_void_p, C.c_size_t, C.c_void_p]),
    "shard_b200_k_quantize_workspace_bytes": (C.c_size_t, [C.c_int32, C.c_int32]),
    "shard_b200_k_quantize_pack": (C.c_int, [C.c_void_p, C.c_void_p, C.c_int32, C.c_int32, C.c_void_p,
                                             C.c_void_p, C.c_void_p, C.c_size_t, C.c_void_p]),
    "shard_b200_int4_pack": (C.c_int, [C.c_void_p, C.c_int64, C.c_void_p, C.c_void_p]),
    "shard_b200_v_hadamard_normalise": (C.c_int, [C.c_void_p, C.c_int64, C.c_int64, C.c_int32, C.c_int32,
                                                  C.c_void_p, C.c_void_p, C.c_void_p]),
    "shard_b200_vq_assign": (C.c_int, [C.c_void_p, C.c_void_p, C.c_int64, C.c_void_p, C.c_void_p, C.c_void_p]),
}

_lib = None


class ShardError(RuntimeError):
    pass


def load():
    """Load the shared library (once) and declare every entry point's signature."""
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(LIB_PATH):
        raise ShardError(
            f"{LIB_PATH} is missing: build it with `python -m shard_b200.build` "
            "(needs nvcc with sm_100a support). There is no CPU fallback.")
    lib = C.CDLL(LIB_PATH)
    for name, (res, args) in _SIGNATURES.items():
        fn = getattr(lib, name)
        fn.restype = res
        fn.argtypes = args
    _lib = lib
    return lib


def symbols():
    return list(_SIGNATURES)


def check(status: int, what: str = "shard_b200 call"):
    if status != 0:
        msg = load().shard_b200_status_string(status).decode()
        raise ShardError(f"{what} failed with status {status}: {msg}")


def ptr(t):
    """Device pointer of a tensor (None -> NULL)."""
    return None if t is None else t.data_ptr()


def cur_stream():
    """Raw handle of the current CUDA stream of the current device."""
    import torch
    try:
        return torch._C._cuda_getCurrentRawStream(torch.cuda.current_device())
    except AttributeError:
        return torch.cuda.current_stream().cuda_stream


def require_cuda(*tensors, current=None):
    """Every tensor must live on the CUDA device that is current: the kernels are launched on
    the current device's current stream with raw pointers, so a tensor of another GPU would be
    read through a wrong (or peer) address.  `current` overrides the device index asked from
    torch (used by tests without a GPU)."""
    cur = current
    for t in tensors:
        if t is None:
            continue
        if not t.is_cuda:
            raise ShardError("shard_b200 kernels need CUDA tensors; there is no CPU fallback")
        if cur is None:
            import torch
            cur = torch.cuda.current_device()
        if t.device.index is not None and t.device.index != cur:
            raise ShardError(f"tensor lives on cuda:{t.device.index} but the current device is cuda:{cur}; "
                             "make the tensor's device current (torch.cuda.device) before the call")
