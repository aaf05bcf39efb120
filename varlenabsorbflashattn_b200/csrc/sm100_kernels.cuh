// tcgen05 / TMA kernels for sm_100a: host-side launchers.
#pragma once
#include "common.cuh"

namespace vafa {

// true when the tcgen05 kernels cover this shape and dtype
bool sm100_varlen_fwd_supported(const vafa_varlen_args* a);
bool sm100_varlen_bwd_supported(const vafa_varlen_args* a);

size_t sm100_varlen_fwd_workspace_bytes(const vafa_varlen_args* a);
size_t sm100_varlen_bwd_workspace_bytes(const vafa_varlen_args* a);
int sm100_varlen_fwd(const vafa_varlen_args* a, cudaStream_t s);
int sm100_varlen_bwd(const vafa_varlen_args* a, cudaStream_t s);
// forward with the library's built-in scratch array instead of a workspace
int sm100_varlen_fwd_noalloc(const vafa_varlen_args* a, cudaStream_t s);

}  // namespace vafa
