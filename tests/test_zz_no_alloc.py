"""The allocation-free decode-attention entry point, called through its exported C symbol.

Some embedders of the library cannot allocate device memory once they are running (all memory
handed to their own arena up front, real-time loops that must stay out of the allocator, hard
memory quotas).  For them the library exports ``mllm_b200_attention_decode_noalloc``, whose only
scratch is a fixed array inside the library image.  This test calls that symbol with raw device
pointers, twice in a row (the second call sees the first call's leftovers in the shared scratch),
and checks both results against the ordinary, allocating op.  It is collected last on purpose.
"""
import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu
D = 128


def _lib():
    from mllm_b200 import _build
    from mllm_b200 import ops

    ops.ext()  # makes sure the extension (and libtorch, which it links) is loaded
    lib = ctypes.CDLL(str(_build._so_path("mllm_b200_C")))
    fn = lib.mllm_b200_attention_decode_noalloc
    fn.restype = ctypes.c_int
    fn.argtypes = [ctypes.c_void_p] * 7 + [ctypes.c_int] * 4 + [ctypes.c_int64] * 3 + [ctypes.c_int, ctypes.c_float,
                                                                                     ctypes.c_int, ctypes.c_void_p]
    lib.mllm_b200_noalloc_last_error.restype = ctypes.c_char_p
    return lib, fn


def _case(seq_lens, hq, hkv, seed):
    torch.manual_seed(seed)
    dev = "cuda"
    B, total = len(seq_lens), sum(seq_lens)
    slots = total + 32
    kc = torch.randn(slots, hkv, D, device=dev, dtype=torch.bfloat16)
    vc = torch.randn(slots, hkv, D, device=dev, dtype=torch.bfloat16)
    rtt = torch.zeros(B + 1, max(seq_lens) + 4, dtype=torch.int32, device=dev)
    perm = torch.randperm(slots - 1, device=dev)[:total].int() + 1
    off = 0
    for b, s in enumerate(seq_lens):
        rtt[b + 1, :s] = perm[off:off + s]
        off += s
    req = torch.arange(1, B + 1, dtype=torch.int32, device=dev)
    seq = torch.tensor(seq_lens, dtype=torch.int32, device=dev)
    q = torch.randn(B, hq, D, device=dev, dtype=torch.bfloat16)
    return q, kc, vc, rtt, req, seq


def _call(fn, q, kc, vc, rtt, req, seq, out, max_len, scale):
    stream = torch.cuda.current_stream().cuda_stream
    return fn(q.data_ptr(), kc.data_ptr(), vc.data_ptr(), rtt.data_ptr(), req.data_ptr(), seq.data_ptr(),
              out.data_ptr(), q.shape[0], q.shape[1], kc.shape[1], D, q.stride(0), rtt.stride(0), kc.shape[0],
              max_len, scale, 0, stream)


def test_no_alloc_decode_matches_allocating_op_twice():
    from mllm_b200 import ops

    lib, fn = _lib()
    scale = D ** -0.5
    for seed, (seq_lens, hq, hkv) in enumerate([([700, 64, 1500, 33], 32, 8), ([2000, 5], 8, 1)]):
        q, kc, vc, rtt, req, seq = _case(seq_lens, hq, hkv, seed)
        want = ops.attention_decode(q, kc, vc, rtt, req, seq, scale, max_seq_len=max(seq_lens))
        for _ in range(2):  # back to back: the second call starts from the first one's scratch contents
            out = torch.full_like(q, float("nan"))
            rc = _call(fn, q, kc, vc, rtt, req, seq, out, max(seq_lens), scale)
            assert rc == 0, lib.mllm_b200_noalloc_last_error().decode()
            torch.cuda.synchronize()
            assert (out.float() - want.float()).abs().max().item() < 3e-2
            assert torch.equal(out, want)  # same kernel, same split: bit-identical
    ops.check_status()


def test_no_alloc_rejects_oversize_and_bad_arguments():
    lib, fn = _lib()
    q, kc, vc, rtt, req, seq = _case([50], 8, 1, 0)
    out = torch.empty_like(q)
    # 16 requests x 128 heads on one KV head with a 1M-token bound -> 8 or more splits x 129 floats each (> 2.1M floats),
    # beyond the 2M-float (8 MiB) array: refused before any launch
    stream = torch.cuda.current_stream().cuda_stream
    rc = fn(q.data_ptr(), kc.data_ptr(), vc.data_ptr(), rtt.data_ptr(), req.data_ptr(), seq.data_ptr(), out.data_ptr(),
            16, 128, 1, D, q.stride(0), rtt.stride(0), kc.shape[0], 1 << 20, 1.0, 0, stream)
    assert rc == 2 and b"scratch" in lib.mllm_b200_noalloc_last_error()
    rc = fn(q.data_ptr(), kc.data_ptr(), vc.data_ptr(), rtt.data_ptr(), req.data_ptr(), seq.data_ptr(), out.data_ptr(),
            1, 8, 1, 64, q.stride(0), rtt.stride(0), kc.shape[0], 50, 1.0, 0, stream)
    assert rc == 1
    rc = fn(None, kc.data_ptr(), vc.data_ptr(), rtt.data_ptr(), req.data_ptr(), seq.data_ptr(), out.data_ptr(),
            1, 8, 1, D, q.stride(0), rtt.stride(0), kc.shape[0], 50, 1.0, 0, stream)
    assert rc == 1
