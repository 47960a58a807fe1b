#include "common.cuh"
namespace ktt {
bool forward_tc5_takes(const AttnParams&, const char** why) { *why = "not built"; return false; }
int launch_forward_tc5(const AttnParams&, cudaStream_t) { return fail(KTT_B200_ERR_UNSUPPORTED, "not built"); }
}
