// Streaming tensor-core expert FFN (placeholder until the kernels land: reports "unsupported"
// so every dispatch takes the generic path).
#include "kernels.h"

bool stream_ffn_supported(int, uint32_t, uint32_t) { return false; }
size_t stream_ffn_scratch_bytes(uint32_t, uint32_t, uint32_t) { return 0; }
cudaError_t launch_ffn_stream(const MoeDispatch &, void *, int, cudaStream_t, int *, cudaEvent_t) { return cudaErrorNotSupported; }
