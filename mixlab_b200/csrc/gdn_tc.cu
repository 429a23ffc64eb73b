// Gated delta rule - tensor-core (tcgen05/TMEM) path for bf16 I/O.
#include "common.cuh"

namespace mxb {

bool gdn_tc_supported(const mxb_gdn_desc*) { return false; }
size_t gdn_tc_workspace_bytes(const mxb_gdn_desc*, bool) { return 0; }
mxb_status gdn_tc_fwd(const mxb_gdn_desc*, const void*, const void*, const void*, const float*,
                      const float*, const float*, void*, float*, void*, cudaStream_t) {
  return MXB_ERR_UNSUPPORTED;
}
mxb_status gdn_tc_bwd(const mxb_gdn_desc*, const void*, const void*, const void*, const float*,
                      const float*, const float*, const void*, const float*, void*, void*, void*,
                      float*, float*, float*, void*, cudaStream_t) {
  return MXB_ERR_UNSUPPORTED;
}

}  // namespace mxb
