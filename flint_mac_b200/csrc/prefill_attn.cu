#include "prefill_attn.h"

namespace flint {
cudaError_t prefill_kernel_setup() { return cudaSuccess; }
cudaError_t launch_prefill(const PrefillParams &, PrefillWorkspace &, cudaStream_t, int *n) { *n = 0; return cudaErrorNotSupported; }
void prefill_workspace_free(PrefillWorkspace &ws) { cudaFree(ws.buf); ws.buf = nullptr; ws.cap = 0; }
}
