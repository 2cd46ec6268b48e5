// placeholder, replaced below
#include "common.cuh"
#include "launch.cuh"
namespace mlstm {
bool sm100_supported(int, int, int, int, int) { return false; }
int sm100_recurrent_fw(const void*, const void*, const GateBuffers&, const float*, const float*, void*, float*, float*, float*, const ChunkwiseDims&, cudaStream_t) { return MLSTM_ERR_UNSUPPORTED; }
int sm100_parallel_fw(const void*, const void*, const void*, const GateBuffers&, const void*, const float*, void*, float*, const ChunkwiseDims&, cudaStream_t) { return MLSTM_ERR_UNSUPPORTED; }
int sm100_recurrent_bw(const void*, const void*, const GateBuffers&, const float*, void*, float*, const ChunkwiseDims&, cudaStream_t) { return MLSTM_ERR_UNSUPPORTED; }
int sm100_parallel_bw(const void*, const void*, const void*, const void*, const GateBuffers&, const void*, const void*, void*, void*, void*, float*, float*, const ChunkwiseDims&, cudaStream_t) { return MLSTM_ERR_UNSUPPORTED; }
}
