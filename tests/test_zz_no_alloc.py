"""The allocation-free convolution entry point (scn_submanifold_convolution_forward_static).

Callers that may not allocate at the point where they run a layer get the tensor-core
convolution with its prepared-weight image in a fixed 8 MiB array inside the library.  This
test calls that entry point straight through the C ABI, twice in a row (the array is shared
and keeps the previous call's image), and checks both results against the regular entry
point, which allocates its image per call, and against the reference's CPU operator.  Around
the two calls neither the library's memory pool nor the device's free memory may move.  It is
collected last on purpose."""
import ctypes as C

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu

TOL = {"tf32": 1e-2, "bf16": 1e-2, "tf32x3": 1e-4}   # the tolerances of the tensor-core tests, per arithmetic mode


def _pool_usage(lib):
    r, u = C.c_uint64(), C.c_uint64()
    assert lib.scn_memory_usage(C.byref(r), C.byref(u)) == 0
    return r.value, u.value


def _ptr(t):
    return C.c_void_p(t.data_ptr())


def test_static_entry_matches_allocating_entry_twice():
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    import sparseconvnet_b200 as scn
    from sparseconvnet_b200._lib import lib, sizes, check
    dev = torch.device("cuda:0")
    torch.cuda.set_device(dev)
    rng = np.random.default_rng(11)
    n = 7000
    pts = rng.integers(0, 56, (n, 2))
    z = (28 + 9 * np.sin(pts[:, 0] / 5.0) + 6 * np.cos(pts[:, 1] / 7.0)).astype(np.int64)
    coords = torch.from_numpy(np.concatenate([pts, z[:, None], rng.integers(0, 2, (n, 1))], axis=1))
    stream = C.c_void_p(torch.cuda.current_stream().cuda_stream)
    size, filt = sizes([56, 56, 56]), sizes([3, 3, 3])
    prec = {"tf32": 1, "bf16": 2, "tf32x3": 3}

    from oracle import runner
    reference = runner.RefBackend() if runner.reference_available() else None
    for (cin, cout), mode in (((32, 64), "tf32"), ((64, 32), "bf16"), ((64, 96), "tf32x3")):
        feats = torch.randn(n, cin, device=dev)
        x = scn.InputLayer(3, 56, mode=4)([coords, feats])
        md = x.metadata._h
        rows = x.features.shape[0]
        weight = (torch.randn(27, 1, cin, cout, device=dev) * 0.1).contiguous()
        bias = torch.randn(cout, device=dev)
        # before the rulebook exists the entry point must refuse rather than build (= allocate) it
        out = torch.empty(rows, cout, device=dev)
        st = lib.scn_submanifold_convolution_forward_static(md, size, filt, _ptr(x.features), _ptr(out), _ptr(weight),
                                                            _ptr(bias), cin, cout, prec[mode], stream)
        assert st == 5 and b"rulebook" in lib.scn_last_error()
        check(lib.scn_md_submanifold_rulebook(md, size, filt, stream, None))

        want = torch.empty(rows, cout, device=dev)
        check(lib.scn_submanifold_convolution_forward(md, size, filt, _ptr(x.features), _ptr(want), _ptr(weight),
                                                      _ptr(bias), cin, cout, 1, prec[mode], stream, None))
        # warm-up call (its first use on the device looks up the array's address), then no allocator may move
        got = torch.full((rows, cout), float("nan"), device=dev)
        check(lib.scn_submanifold_convolution_forward_static(md, size, filt, _ptr(x.features), _ptr(got), _ptr(weight),
                                                             _ptr(bias), cin, cout, prec[mode], stream))
        torch.cuda.synchronize()
        for call in range(2):
            got.fill_(float("nan"))
            torch.cuda.synchronize()
            pool_before, free_before = _pool_usage(lib), torch.cuda.mem_get_info()[0]
            check(lib.scn_submanifold_convolution_forward_static(md, size, filt, _ptr(x.features), _ptr(got),
                                                                 _ptr(weight), _ptr(bias), cin, cout, prec[mode],
                                                                 stream))
            torch.cuda.synchronize()
            assert _pool_usage(lib) == pool_before and torch.cuda.mem_get_info()[0] == free_before, \
                "the allocation-free entry point moved an allocator"
            check(lib.scn_md_poll_errors(md, stream))
            err = float((got - want).abs().max() / want.abs().max())
            assert err <= TOL[mode], "%s call %d: relative difference %.3g" % (mode, call, err)
            if reference is not None:  # and against the reference's own CPU operator on the same rows
                import types
                xo = runner.OTensor(x.features.cpu().numpy(), None, [56, 56, 56])
                md_ref = reference.input_layer(3, [56, 56, 56], 4, coords.numpy(), feats.cpu().numpy(), 0)
                xo.metadata = md_ref.metadata
                assert np.array_equal(reference.locations(md_ref), x.get_spatial_locations().numpy())
                yo, _ = reference.subconv(xo, [3, 3, 3], weight.cpu(), bias.cpu())
                err = float(np.abs(got.cpu().numpy() - yo.features).max() / np.abs(yo.features).max())
                assert err <= TOL[mode], "%s call %d vs reference: relative difference %.3g" % (mode, call, err)
            # a different weight in between makes sure the second call does not live off the first image
            weight = (weight * 1.5).contiguous()
            check(lib.scn_submanifold_convolution_forward(md, size, filt, _ptr(x.features), _ptr(want), _ptr(weight),
                                                          _ptr(bias), cin, cout, 1, prec[mode], stream, None))

    # beyond the built-in buffer: 27 * 256 * 256 * 8 bytes (tf32x3 as two tf32 parts) = 13.5 MiB > 8 MiB
    import os
    os.environ["SCN_X3_FORM"] = "tf32"
    feats = torch.randn(n, 256, device=dev)
    x = scn.InputLayer(3, 56, mode=4)([coords, feats])
    check(lib.scn_md_submanifold_rulebook(x.metadata._h, size, filt, stream, None))
    big = torch.zeros(27, 1, 256, 256, device=dev)
    out = torch.empty(x.features.shape[0], 256, device=dev)
    st = lib.scn_submanifold_convolution_forward_static(x.metadata._h, size, filt, _ptr(x.features), _ptr(out),
                                                        _ptr(big), None, 256, 256, prec["tf32x3"], stream)
    del os.environ["SCN_X3_FORM"]
    assert st == 7 and b"8388608" in lib.scn_last_error()
    # precision fp32 has no tensor-core kernel: refused, not silently redirected
    st = lib.scn_submanifold_convolution_forward_static(x.metadata._h, size, filt, _ptr(x.features), _ptr(out),
                                                        _ptr(big), None, 256, 256, 0, stream)
    assert st == 7
