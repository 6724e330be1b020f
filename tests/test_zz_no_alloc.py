"""The allocation-free CSR entry point, called through its exported C symbol.

``clt_build_csr_static`` serves embedders that may not allocate device memory (a host process that owns the
whole memory budget, a sandboxed plugin, a latency-critical path that cannot afford cudaMalloc's implicit
synchronisation).  It must give exactly what ``clt_build_csr`` gives with caller-provided scratch.  Two calls
in a row on different inputs also check that the library-resident scratch, which keeps the previous call's
contents, is cleared where it has to start from zero.  The file name makes pytest collect it last.
"""
import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu


def _make_entries(seed, n, num_tokens, num_layers, col_pitch, dev):
    g = torch.Generator().manual_seed(seed)
    flat = torch.randperm(num_tokens * num_layers * col_pitch, generator=g)[:n]  # unique (token, column) pairs
    tok = (flat // (num_layers * col_pitch)).to(torch.int32)
    col = (flat % (num_layers * col_pitch)).to(torch.int32)
    val = torch.randn(n, generator=g)
    ctl = torch.zeros(16, dtype=torch.int64)
    ctl[3] = n
    return tok.to(dev), col.to(dev), val.to(dev), ctl.to(dev)


def _alloc_outputs(cap, num_tokens, num_cols, dev):
    i32, f32 = torch.int32, torch.float32
    return dict(
        tok_off=torch.zeros(num_tokens + 1, dtype=i32, device=dev), feat_off=torch.zeros(num_cols + 1, dtype=i32, device=dev),
        tcsr_col=torch.zeros(cap, dtype=i32, device=dev), tcsr_val=torch.zeros(cap, dtype=f32, device=dev),
        fcsr_tok=torch.zeros(cap, dtype=i32, device=dev), fcsr_val=torch.zeros(cap, dtype=f32, device=dev),
    )


def test_static_csr_matches_regular_entry_point_twice():
    from crosslayer_coding_b200.ops import ext as ext_mod

    ext = ext_mod.load()
    lib = ctypes.CDLL(ext_mod.so_file())
    fn = lib.clt_build_csr_static
    fn.restype = ctypes.c_int
    vp, ll, ci = ctypes.c_void_p, ctypes.c_longlong, ctypes.c_int
    fn.argtypes = [vp, vp, vp, ll, vp, ci, ci, ci, vp, vp, vp, vp, vp, vp, ci, vp]
    dev = torch.device("cuda:0")
    torch.cuda.set_device(dev)
    num_tokens, num_layers, col_pitch = 96, 3, 160
    num_cols = num_layers * col_pitch
    stream = torch.cuda.current_stream().cuda_stream
    for seed, n in ((1, 900), (2, 350)):  # the second call sees the first call's leftovers in the scratch
        tok, col, val, ctl = _make_entries(seed, n, num_tokens, num_layers, col_pitch, dev)
        cap = n
        want = _alloc_outputs(cap, num_tokens, num_cols, dev)
        i32 = torch.int32
        scratch = [torch.zeros(num_tokens, dtype=i32, device=dev), torch.zeros(num_cols, dtype=i32, device=dev),
                   torch.zeros(num_tokens, dtype=i32, device=dev), torch.zeros(num_cols, dtype=i32, device=dev)]
        ext.build_csr(tok, col, val, ctl, num_tokens, num_cols, scratch[0], scratch[1], want["tok_off"], want["feat_off"],
                      scratch[2], scratch[3], want["tcsr_col"], want["tcsr_val"], want["fcsr_tok"], want["fcsr_val"], None, 3, col_pitch)
        got = _alloc_outputs(cap, num_tokens, num_cols, dev)
        rc = fn(tok.data_ptr(), col.data_ptr(), val.data_ptr(), cap, ctl.data_ptr(), num_tokens, num_cols, col_pitch,
                got["tok_off"].data_ptr(), got["feat_off"].data_ptr(), got["tcsr_col"].data_ptr(), got["tcsr_val"].data_ptr(),
                got["fcsr_tok"].data_ptr(), got["fcsr_val"].data_ptr(), 3, stream)
        assert rc == 0
        torch.cuda.synchronize()
        for name in want:
            assert torch.equal(got[name], want[name]), name
        assert int(got["tok_off"][-1]) == n and int(got["feat_off"][-1]) == n


def test_static_csr_rejects_oversized_problems():
    from crosslayer_coding_b200.ops import ext as ext_mod

    ext_mod.load()
    lib = ctypes.CDLL(ext_mod.so_file())
    fn = lib.clt_build_csr_static
    fn.restype = ctypes.c_int
    vp, ll, ci = ctypes.c_void_p, ctypes.c_longlong, ctypes.c_int
    fn.argtypes = [vp, vp, vp, ll, vp, ci, ci, ci, vp, vp, vp, vp, vp, vp, ci, vp]
    dev = torch.device("cuda:0")
    t = torch.zeros(64, dtype=torch.int32, device=dev)
    f = torch.zeros(64, dtype=torch.float32, device=dev)
    ctl = torch.zeros(16, dtype=torch.int64, device=dev)
    p = t.data_ptr()
    too_many_cols = (1 << 20) + 1
    rc = fn(p, p, f.data_ptr(), 64, ctl.data_ptr(), 16, too_many_cols, 1024, p, p, p, f.data_ptr(), p, f.data_ptr(), 0, None)
    assert rc == -2
    rc = fn(p, p, f.data_ptr(), 64, ctl.data_ptr(), 0, 16, 16, p, p, p, f.data_ptr(), p, f.data_ptr(), 0, None)
    assert rc == -1
