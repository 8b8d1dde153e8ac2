"""``nms3d`` and ``yolox3d_decode`` (deploy3d/symfun/ops/decoder/nms3d.py, yolox3d_decode.py)."""
import numpy as np

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


def data_s_yolox3d_decode(stride, class_ids, topk):
    """The blob the reference exporter writes (deploy3d/symfun/ops/decoder/yolox3d_decode.py:43-50)."""
    class_ids = tuple(int(c) for c in class_ids)
    assert len(class_ids) <= 8
    return (np.array([stride, topk], dtype=np.int32).tobytes() +
            np.array(class_ids + (-1,) * (8 - len(class_ids)), dtype=np.int32).tobytes())


def yolox3d_decode(cls_scores, bbox_preds, voxel_config, stride, class_ids, topk):
    """cls_scores [B, C, Y, X], bbox_preds [B, 9+a, Y, X] (same dtype), voxel_config float32 [6]; returns
    (topk_class_ids, topk_scores, topk_boxes) for every class id, in order
    (deploy3d/symfun/ops/decoder/yolox3d_decode.py:20-37)."""
    plug = _plugin("YoloX3dDecode", data_s_yolox3d_decode(stride, class_ids, topk))
    return plug.enqueue(cls_scores, bbox_preds, voxel_config)
