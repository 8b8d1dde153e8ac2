// Library identification and status strings.
#include "common.cuh"

extern "C" const char* d3d_version(void) { return "deploy3d_b200 0.1 (sm_100a)"; }

extern "C" const char* d3d_status_string(int status) {
  switch (status) {
    case D3D_OK: return "ok";
    case D3D_ERR_INVALID_ARGUMENT: return "invalid argument";
    case D3D_ERR_UNSUPPORTED_DTYPE: return "unsupported dtype";
    case D3D_ERR_WORKSPACE_TOO_SMALL: return "workspace too small";
    case D3D_ERR_CUDA: return "CUDA error";
    case D3D_ERR_BAD_BLOB: return "truncated or malformed data_s blob";
    case D3D_ERR_TOO_LARGE: return "problem exceeds an implementation limit";
    default: return "unknown status";
  }
}
