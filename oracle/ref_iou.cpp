// TEST INFRASTRUCTURE ONLY.  Thin C wrapper that compiles the reference's own
// trt/decoder/iou_rotated.cuh for the host (it is plain C++ once HOST_DEVICE_INLINE
// degrades to `inline`, see trt/include/common/macros.h:36-40).  The resulting
// oracle/_ref/libref_iou.so is used to pin oracle.c's restatement of the rotated-IoU
// arithmetic bit for bit.  The reference sources are read where they lie; nothing is copied.
#include <cmath>
#include <cstdio>
using std::fabs;
#include "decoder/iou_rotated.cuh"

extern "C" float ref_rotated_intersection(float cx1, float cy1, float w1, float h1, float a1, float cx2, float cy2,
                                          float w2, float h2, float a2) {
  iou_rotated::RotatedBox<float> b1{cx1, cy1, w1, h1, a1}, b2{cx2, cy2, w2, h2, a2};
  return iou_rotated::rotated_boxes_intersection<float>(b1, b2);
}

// trt/decoder/nms3d.cu:32-56 restated around the reference intersection.
extern "C" float ref_bev_iou(const float* a, const float* b) {
  float va = a[3] * a[4], vb = b[3] * b[4];
  float ov = ref_rotated_intersection(a[0], a[1], a[3], a[4], a[6], b[0], b[1], b[3], b[4], b[6]);
  return ov / fmaxf(va + vb - ov, iou_rotated::EPS);
}
