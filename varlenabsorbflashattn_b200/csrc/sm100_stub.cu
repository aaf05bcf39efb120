#include "sm100_kernels.cuh"
namespace vafa {
bool sm100_varlen_bwd_supported(const vafa_varlen_args*) { return false; }
size_t sm100_varlen_bwd_workspace_bytes(const vafa_varlen_args*) { return 0; }
int sm100_varlen_bwd(const vafa_varlen_args*, cudaStream_t) { return fail(VAFA_ERR_UNSUPPORTED, "not built"); }
}
