"""NMS3d for hosts that cannot allocate: d3d_nms3d_enqueue_static keeps its scratch inside the library.

Some users of the library own nothing but input/output pointers and a stream -- a real-time loop that bans device
allocation once it runs, an engine built without plugin workspace -- so they cannot hand NMS3d the mask workspace
the regular entry point wants.  The static variant must give exactly the same scores, call after call (the shared
scratch keeps the previous call's contents), and must refuse problems larger than its fixed scratch.

Collected last on purpose (file name): a run that stops at the first failure has then already run every other test.
"""
import ctypes

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _call_both(lib, _lib, scores, boxes, thr):
    """Runs the workspace entry point and the static one through the C ABI; returns both outputs."""
    p = _lib.Nms3dParams(thr)
    ins = [_lib.make_desc(_lib.D3D_FLOAT, tuple(scores.shape)), _lib.make_desc(_lib.D3D_FLOAT, tuple(boxes.shape))]
    outs = [_lib.make_desc(_lib.D3D_FLOAT, tuple(scores.shape))]
    in_ptrs = _lib.ptr_array([scores.data_ptr(), boxes.data_ptr()])
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    nbytes = ctypes.c_size_t(0)
    _lib.check("workspace", lib.d3d_nms3d_workspace(ctypes.byref(p), _lib.desc_array(ins), 2, ctypes.byref(nbytes)))
    ws = torch.empty(max(nbytes.value, 16), dtype=torch.uint8, device=DEV)
    want = torch.full_like(scores, 7.0)
    _lib.check("enqueue", lib.d3d_nms3d_enqueue(ctypes.byref(p), _lib.desc_array(ins), 2, _lib.desc_array(outs), 1,
                                                in_ptrs, _lib.ptr_array([want.data_ptr()]),
                                                ctypes.c_void_p(ws.data_ptr()), nbytes, stream))
    got = torch.full_like(scores, 9.0)
    torch.cuda.synchronize()
    free_before = torch.cuda.mem_get_info()[0]
    status = lib.d3d_nms3d_enqueue_static(ctypes.byref(p), _lib.desc_array(ins), 2, _lib.desc_array(outs), 1, in_ptrs,
                                          _lib.ptr_array([got.data_ptr()]), stream)
    _lib.check("enqueue_static", status)
    assert torch.cuda.mem_get_info()[0] >= free_before  # the call took no device memory from the driver
    torch.cuda.synchronize()
    return want.cpu().numpy(), got.cpu().numpy()


def test_static_scratch_matches_workspace_variant_twice(d3d):
    from deploy3d_b200 import _lib, synth
    lib = _lib.lib()
    big = synth.config4_boxes(10, 1000)         # 160 000 mask words: the largest benchmark case
    small = synth.config4_boxes(3, 200)         # a smaller second call must not see the first one's leftovers
    small["boxes"][..., :2] *= 0.1               # crowded: most boxes are suppressed
    for case, thr in ((big, 0.2), (small, 0.1), (big, 0.1)):
        scores = torch.from_numpy(case["scores"]).to(DEV)
        boxes = torch.from_numpy(case["boxes"]).to(DEV)
        want, got = _call_both(lib, _lib, scores, boxes, thr)
        assert (want == got).all()
        assert ((got == -1) | (got == case["scores"])).all() and (got >= 0).any()


def test_static_scratch_refuses_oversized_problems(d3d):
    from deploy3d_b200 import _lib
    lib = _lib.lib()
    b, k = 3, 4096                               # 3 * 4096 * 64 words > 256 Ki
    scores = torch.zeros((b, k), device=DEV)
    boxes = torch.zeros((b, k, 7), device=DEV)
    p = _lib.Nms3dParams(0.1)
    ins = [_lib.make_desc(_lib.D3D_FLOAT, (b, k)), _lib.make_desc(_lib.D3D_FLOAT, (b, k, 7))]
    outs = [_lib.make_desc(_lib.D3D_FLOAT, (b, k))]
    out = torch.full((b, k), 5.0, device=DEV)
    status = lib.d3d_nms3d_enqueue_static(ctypes.byref(p), _lib.desc_array(ins), 2, _lib.desc_array(outs), 1,
                                          _lib.ptr_array([scores.data_ptr(), boxes.data_ptr()]),
                                          _lib.ptr_array([out.data_ptr()]),
                                          ctypes.c_void_p(torch.cuda.current_stream().cuda_stream))
    assert status == -6  # D3D_ERR_TOO_LARGE
    torch.cuda.synchronize()
    assert (out == 5.0).all()  # nothing ran
