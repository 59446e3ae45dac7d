"""The allocation-free C entry point, called the way its intended users call it: through the
exported C symbol of the torch-free shared library, with every buffer supplied by the caller.

Some hosts of this library may not allocate device memory while they run (a plugin inside a
pipeline whose memory was handed out up front, a real-time loop that must not touch the
allocator).  For them ``hipress_terngrad_compress_noalloc`` keeps its reduction scratch in a
fixed device array inside the library.  Its payload must equal the regular op's byte for byte,
on the first call and on a second call that finds the scratch as the first one left it.
"""
import ctypes
import os

import pytest
import torch

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _lib():
    import hipress_b200  # noqa: F401  (makes sure the libraries are built)
    lib = ctypes.CDLL(os.path.join(ROOT, "hipress_b200", "libhipress_kernels.so"))
    fn = lib.hipress_terngrad_compress_noalloc
    fn.restype = ctypes.c_int
    fn.argtypes = [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_longlong, ctypes.c_int, ctypes.c_int,
                   ctypes.c_ulonglong, ctypes.c_void_p, ctypes.c_longlong, ctypes.c_void_p]
    lib.hipress_noalloc_last_error.restype = ctypes.c_char_p
    return lib, fn


def test_noalloc_terngrad_matches_regular_entry_point_twice():
    from hipress_b200 import ops
    lib, fn = _lib()
    torch.cuda.set_device(0)
    stream = torch.cuda.current_stream().cuda_stream
    for call, (n, bw, seed) in enumerate([(1_000_003, 2, 11), (262_144 + 5, 4, 12)]):
        g = (torch.randn(n, generator=torch.Generator().manual_seed(call)) * 0.01).cuda()
        r0 = (torch.randn(n, generator=torch.Generator().manual_seed(100 + call)) * 0.002).cuda()
        # existing entry point
        r_ref = r0.clone()
        ref = ops.terngrad_compress(g, bw, True, seed, residual=r_ref)
        # new entry point: caller-owned buffers only
        r_new = r0.clone()
        out = torch.empty(ops.terngrad_payload_bytes(n, bw), dtype=torch.uint8, device="cuda")
        rc = fn(g.data_ptr(), r_new.data_ptr(), n, bw, 1, seed, out.data_ptr(), out.numel(), stream)
        assert rc == 0, lib.hipress_noalloc_last_error()
        torch.cuda.synchronize()
        assert torch.equal(out, ref), f"payload differs on call {call}"
        assert torch.equal(r_new, r_ref), f"residual differs on call {call}"


def test_noalloc_without_residual_and_with_4_byte_aligned_buffers():
    """No residual, and gradient / residual that are 4-byte but not 16-byte aligned (a view one
    element into a tensor): the scalar-load forms of the kernels, through the same entry."""
    from hipress_b200 import ops
    lib, fn = _lib()
    stream = torch.cuda.current_stream().cuda_stream
    n, bw, seed = 300_001, 2, 21
    base = (torch.randn(n + 1, generator=torch.Generator().manual_seed(5)) * 0.01).cuda()
    rbase = (torch.randn(n + 1, generator=torch.Generator().manual_seed(6)) * 0.002).cuda()
    for g, r0 in ((base[:n], None), (base[1:], None), (base[1:], rbase[1:])):
        r_ref = None if r0 is None else r0.clone()
        ref = ops.terngrad_compress(g.clone(), bw, True, seed, residual=r_ref)
        # a clone is freshly aligned: rebuild the one-element offset for the new entry point
        holder = torch.empty(n + 1, device="cuda")
        off = 1 if g.data_ptr() % 16 else 0
        g_new = holder[off:off + n]
        g_new.copy_(g)
        assert g_new.data_ptr() % 16 == g.data_ptr() % 16
        r_new = None
        if r0 is not None:
            rholder = torch.empty(n + 1, device="cuda")
            r_new = rholder[1:1 + n]
            r_new.copy_(r0)
        out = torch.empty(ops.terngrad_payload_bytes(n, bw), dtype=torch.uint8, device="cuda")
        rc = fn(g_new.data_ptr(), None if r_new is None else r_new.data_ptr(), n, bw, 1, seed, out.data_ptr(),
                out.numel(), stream)
        assert rc == 0, lib.hipress_noalloc_last_error()
        torch.cuda.synchronize()
        assert torch.equal(out, ref)
        if r0 is not None:
            assert torch.equal(r_new, r_ref)


def test_noalloc_rejects_bad_sizes():
    lib, fn = _lib()
    g = torch.zeros(16, device="cuda")
    out = torch.zeros(14, dtype=torch.uint8, device="cuda")
    assert fn(g.data_ptr(), None, 16, 2, 0, 0, out.data_ptr(), 13, None) == 1          # wrong out_bytes
    assert fn(g.data_ptr(), None, 16, 3, 0, 0, out.data_ptr(), 14, None) == 1          # bad bitwidth
    assert fn(g.data_ptr(), None, (1 << 31), 2, 0, 0, out.data_ptr(), 14, None) == 2   # beyond the maximum
    assert b"MAX_ELEMS" in lib.hipress_noalloc_last_error()
