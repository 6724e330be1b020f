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


def test_static_csr_skips_out_of_range_entries_and_handles_the_size_limits():
    """Entries outside the problem are left out of both views (nothing is written outside this call's regions), and a
    problem at the documented limits (65 536 tokens, 1 048 576 columns) goes through."""
    from crosslayer_coding_b200.ops import ext as ext_mod

    ext_mod.load()
    lib = ctypes.CDLL(ext_mod.so_file())
    fn = lib.clt_build_csr_static
    fn.restype = ctypes.c_int
    vp, ll, ci = ctypes.c_void_p, ctypes.c_longlong, ctypes.c_int
    fn.argtypes = [vp, vp, vp, ll, vp, ci, ci, ci, vp, vp, vp, vp, vp, vp, ci, vp]
    dev = torch.device("cuda:0")
    torch.cuda.set_device(dev)
    stream = torch.cuda.current_stream().cuda_stream

    def call(tok, col, val, ctl, num_tokens, num_cols, col_pitch):
        out = _alloc_outputs(tok.numel(), num_tokens, num_cols, dev)
        rc = fn(tok.data_ptr(), col.data_ptr(), val.data_ptr(), tok.numel(), ctl.data_ptr(), num_tokens, num_cols, col_pitch,
                out["tok_off"].data_ptr(), out["feat_off"].data_ptr(), out["tcsr_col"].data_ptr(), out["tcsr_val"].data_ptr(),
                out["fcsr_tok"].data_ptr(), out["fcsr_val"].data_ptr(), 3, stream)
        torch.cuda.synchronize()
        return rc, out

    num_tokens, num_layers, col_pitch = 40, 2, 64
    tok, col, val, ctl = _make_entries(5, 200, num_tokens, num_layers, col_pitch, dev)
    good_rc, good = call(tok, col, val, ctl, num_tokens, num_layers * col_pitch, col_pitch)
    bad_tok, bad_col = tok.clone(), col.clone()
    bad_tok[7] = num_tokens + 3          # token beyond the problem
    bad_col[11] = num_layers * col_pitch  # first column beyond the problem
    bad_col[13] = -1
    rc, got = call(bad_tok, bad_col, val, ctl, num_tokens, num_layers * col_pitch, col_pitch)
    assert good_rc == 0 and rc == 0
    assert int(got["tok_off"][-1]) == 197 and int(got["feat_off"][-1]) == 197
    keep = torch.ones(200, dtype=torch.bool, device=dev)
    keep[[7, 11, 13]] = False
    ctl2 = ctl.clone()
    ctl2[3] = 197
    rc, want = call(tok[keep].contiguous(), col[keep].contiguous(), val[keep].contiguous(), ctl2, num_tokens, num_layers * col_pitch, col_pitch)
    for name in ("tok_off", "feat_off"):
        assert torch.equal(got[name], want[name]), name
    for name in ("tcsr_col", "tcsr_val", "fcsr_tok", "fcsr_val"):
        assert torch.equal(got[name][:197], want[name][:197]), name
    # at the limits
    T, C = 65536, 1 << 20
    g = torch.Generator().manual_seed(9)
    n = 5000
    tok = torch.randint(0, T, (n,), generator=g).to(torch.int32).to(dev)
    col = torch.randperm(C, generator=g)[:n].to(torch.int32).to(dev)
    tok[0], col[0] = T - 1, C - 1
    val = torch.randn(n, generator=g).to(dev)
    ctl = torch.zeros(16, dtype=torch.int64, device=dev)
    ctl[3] = n
    rc, out = call(tok, col, val, ctl, T, C, 1 << 16)
    assert rc == 0 and int(out["tok_off"][-1]) == n and int(out["feat_off"][-1]) == n
    cnt = torch.bincount(tok.long(), minlength=T)
    assert torch.equal(out["tok_off"][1:].long() - out["tok_off"][:-1].long(), cnt)
    assert int(out["feat_off"][C]) - int(out["feat_off"][C - 1]) == 1
