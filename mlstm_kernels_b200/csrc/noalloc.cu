// Forward entry point for hosts that must not allocate device memory.
//
// Some embedders cannot call cudaMalloc (or any allocator built on it) once they are up: serving runtimes
// that hand every free byte of the GPU to their own pool at start-up, so that a later driver allocation
// simply fails, and hot loops that ban allocator calls because of their unpredictable latency.  The regular
// forward wants a caller-provided workspace, which such a host would have had to reserve in advance; this
// variant carries its workspace inside the library instead, as a fixed-size array in device global memory
// that exists as long as the library is loaded (every GPU that loads the library holds a copy).
#include <mutex>

#include "common.cuh"
#include "launch.cuh"

namespace {

constexpr size_t kStaticScratchBytes = 8u << 20;  // 8 MiB, enough for about 400k (batch x head x token) units
__device__ __align__(256) unsigned char g_static_scratch[kStaticScratchBytes];

constexpr int kMaxDevices = 64;
std::mutex g_mu;
void* g_scratch_ptr[kMaxDevices] = {};  // device address of g_static_scratch, one per device ordinal

// Host code cannot use the array's name as a pointer (it is a host-side shadow symbol, not a device address):
// ask the runtime for the real address once per device, with that device current.
int scratch_for_current_device(void** out) {
  int dev = -1;
  MLSTM_CUDA_CHECK(cudaGetDevice(&dev));
  if (dev < 0 || dev >= kMaxDevices) return MLSTM_ERR_UNSUPPORTED;
  std::lock_guard<std::mutex> lk(g_mu);
  if (g_scratch_ptr[dev] == nullptr) {
    void* p = nullptr;
    MLSTM_CUDA_CHECK(cudaGetSymbolAddress(&p, g_static_scratch));
    g_scratch_ptr[dev] = p;
  }
  *out = g_scratch_ptr[dev];
  return MLSTM_OK;
}

// The scratch address belongs to the CURRENT device; a stream of another device would make the kernels of that
// device write through a pointer that means something else there.  Refuse the mismatch where the runtime can tell.
int check_stream_on_current_device(void* stream) {
  int cur = -1, sdev = -1;
  MLSTM_CUDA_CHECK(cudaGetDevice(&cur));
  if (cudaStreamGetDevice(static_cast<cudaStream_t>(stream), &sdev) != cudaSuccess) {
    (void)cudaGetLastError();   // the query is unavailable for this stream: nothing to compare
    return MLSTM_OK;
  }
  return sdev == cur ? MLSTM_OK : MLSTM_ERR_UNSUPPORTED;
}

}  // namespace

extern "C" {

size_t mlstm_b200_static_scratch_bytes(void) { return kStaticScratchBytes; }

int mlstm_b200_static_warmup(void) {
  void* scratch = nullptr;
  int rc = scratch_for_current_device(&scratch);   // materialises the array on this device
  if (rc != MLSTM_OK) return rc;
  if ((rc = mlstm::gates_force_load()) != MLSTM_OK) return rc;
  return mlstm::sm100_force_load();
}

int mlstm_b200_chunkwise_fw_static(const void* q, const void* k, const void* v, const void* i, const void* f,
                                   const float* c_initial, const float* n_initial, const float* m_initial, void* h,
                                   float* n_out, float* m_out, void* c_states, float* n_states, float* m_states,
                                   float* c_last, float* n_last, float* m_last, int B, int NH, int S, int DHQK,
                                   int DHHV, int L, int dtype, int gate_dtype, int variant, int impl, float eps,
                                   void* stream) {
  const size_t need = mlstm_b200_chunkwise_workspace_bytes(B, NH, S, DHQK, DHHV, L, dtype, variant, impl, 0);
  if (need == 0) return MLSTM_ERR_SHAPE;
  if (need > kStaticScratchBytes) return MLSTM_ERR_WORKSPACE;  // problem too large for the built-in scratch
  void* scratch = nullptr;
  int rc = check_stream_on_current_device(stream);
  if (rc != MLSTM_OK) return rc;
  if ((rc = scratch_for_current_device(&scratch)) != MLSTM_OK) return rc;
  // The forward writes every scratch word before it reads it, so nothing has to be cleared between calls.
  // Single-stream form of the forward: the two-stream split of the regular entry point would create a stream and two
  // events on its first use, which is driver memory this entry point promises not to take.
  return mlstm::chunkwise_fw_body(q, k, v, i, f, c_initial, n_initial, m_initial, h, n_out, m_out, c_states, n_states,
                                  m_states, c_last, n_last, m_last, scratch, kStaticScratchBytes, B, NH, S, DHQK, DHHV,
                                  L, dtype, gate_dtype, variant, impl, eps, stream, false);
}

}  // extern "C"
