// placeholder replaced below
#include "common.cuh"
#include "spconv_mm_internal.h"
namespace d3d {
bool spconv_mm_tc_eligible(const d3d_spconv_mm_s*, int) { return false; }
int launch_spconv_mm_tc(const MmLaunch&) { return D3D_ERR_INVALID_ARGUMENT; }
void spconv_mm_tc_release(d3d_spconv_mm_s*) {}
}  // namespace d3d
