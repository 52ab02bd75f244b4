// tcgen05 kernels — placeholder while the first path is brought up.
#include "common.cuh"
namespace mintb {
bool tc_supported(int, int) { return false; }
size_t tc_fwd_workspace_bytes(int, int, int, int, bool) { return 0; }
size_t tc_bwd_workspace_bytes(int, int, int, int, bool) { return 0; }
int launch_attn_fwd_tc(const AttnArgs&) { set_error("tcgen05 path not built"); return MINTB_EUNSUPPORTED; }
int launch_attn_bwd_tc(const AttnArgs&) { set_error("tcgen05 path not built"); return MINTB_EUNSUPPORTED; }
}
