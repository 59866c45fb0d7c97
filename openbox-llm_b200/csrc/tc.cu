// placeholder until the tcgen05 kernels land
#include "common.cuh"
namespace nsa {
bool tc_shape_ok(const NsaDims&, int) { return false; }
int tc_attn_fwd(const AttnArgs&, cudaStream_t) { set_error("tc path not built"); return NSA_ERR_UNSUPPORTED; }
size_t tc_attn_bwd_workspace(const AttnArgs&) { return 0; }
int tc_attn_bwd(const AttnArgs&, void*, size_t, cudaStream_t) { set_error("tc path not built"); return NSA_ERR_UNSUPPORTED; }
}
