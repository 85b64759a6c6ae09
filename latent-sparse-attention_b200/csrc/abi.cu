// Error names and the ABI version of the library.
#include "common.cuh"

LSA_API const char *lsa_error_string(int code) {
  switch (code) {
    case LSA_OK: return "ok";
    case LSA_ERR_ARGUMENT: return "a size, stride or combination of arguments the kernels do not take";
    case LSA_ERR_NULL: return "a required pointer is NULL";
    case LSA_ERR_UNSUPPORTED: return "a shape outside what the kernels were written for";
    case LSA_ERR_WORKSPACE: return "the workspace is smaller than the matching *_workspace_bytes() asks";
    case LSA_ERR_LAUNCH: return "the CUDA runtime refused a launch or a kernel attribute";
    case LSA_ERR_DEVICE: return "the current device is not an sm_100 GPU";
    case LSA_ERR_STATIC_SCRATCH:
      return "the call needs more scratch than the 8 MiB static array of lsa_sparse_attend_static holds - lower splits or rows";
    default: return "unknown lsa_b200 error code";
  }
}

LSA_API int lsa_abi_version(void) { return 18; }
