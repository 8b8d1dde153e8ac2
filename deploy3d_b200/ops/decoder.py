"""``nms3d`` (deploy3d/symfun/ops/decoder/nms3d.py)."""
from .spconv import _plugin


def nms3d(scores, boxes, iou_threshold=None):
    """scores [B, K] sorted descending, boxes [B, K, 7+a]; suppressed scores become -1.

    The reference plugin has no parameters and a fixed IoU threshold of 0.1 (trt/decoder/nms3d.cu:138);
    ``iou_threshold`` overrides it for callers that go through this module."""
    plug = _plugin("NMS3d", b"")
    if iou_threshold is not None:
        import copy
        plug = copy.copy(plug)
        plug.p = type(plug.p)(float(iou_threshold))
        plug._workspace = None
    return plug.enqueue(scores, boxes)[0]
