// Registration of the standalone ops (normalisation, quantisation, RoPE, activation), the
// tcgen05 GEMMs, the fused GEMM+collective ops and the decode-attention kernel.
#include "tdx/bindings.h"

namespace tdx_torch {

void register_extra_ops(torch::Library& m) { (void)m; }

}  // namespace tdx_torch
