// placeholder, replaced below
#include "../../include/fmha_sm100.h"
#include "fmha_kernel_args.h"
namespace fmha { int launch_bwd(const BwdArgs&, int, int, cudaStream_t) { return 1; } }
extern "C" int fmha_sm100_bwd(const fmha_bwd_params*, void*) { return FMHA_ERR_UNSUPPORTED; }
extern "C" int fmha_sm100_bwd_workspace_bytes(const fmha_bwd_params*, size_t*) { return FMHA_ERR_UNSUPPORTED; }
