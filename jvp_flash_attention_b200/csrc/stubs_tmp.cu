#include "host_common.h"
namespace jvpfa {
int launch_fwd_generic(const jvpfa_fwd_args&, cudaStream_t) { return JVPFA_ERR_UNSUPPORTED; }
int launch_bwd_generic(const jvpfa_bwd_args&, cudaStream_t) { return JVPFA_ERR_UNSUPPORTED; }
size_t bwd_generic_workspace_bytes(const jvpfa_bwd_args&) { return kStatusBytes; }
}
