// Host-side launcher prototypes shared between the translation units of libmlstm_b200.so.
#pragma once
#include "common.cuh"

namespace mlstm {

// gates.cu
// m_out (nullable): user-visible copy of the per-token max state, S entries per (batch, head)
int launch_gates(int dtype, const void* i, const void* f, const float* m_initial, const float* n_out, float* m_out,
                 const GateBuffers& gb, float* m_states, const ChunkwiseDims& d, cudaStream_t st,
                 float m_default = 0.f, float* g_sum = nullptr);
int launch_inv_den(const float* n_out, float* inv_den, const ChunkwiseDims& d, cudaStream_t st);
int launch_state_combine(const float* c_in, const float* n_in, const float* m_in, const float* c_loc,
                         const float* n_loc, const float* m_loc, const float* g_total, float* c_out, float* n_out,
                         float* m_out, int BNH, int DHQK, int DHHV, int variant, cudaStream_t st);
int launch_gate_grads(int dtype, int gate_dtype, const void* q, const void* k, const void* dq, const void* dk, const void* i,
                      const void* f, float* acc, float* kdk, float* dI, float* dF, const ChunkwiseDims& d,
                      cudaStream_t st);
int launch_gate_grad_scan(int dtype, const void* i, const void* f, const float* qdq, const float* kdk, int nparts,
                          float* dI, float* dF, const ChunkwiseDims& d, cudaStream_t st, const float* anchors,
                          int n_anchors, int anchor_tokens);
int launch_state_dot(const void* c_states, const void* dc_states, float* anchors, int every, int n_anchors,
                     const ChunkwiseDims& d, cudaStream_t st);

// chunkwise_simt.cu : portable CUDA-core kernels, any shape, any element type
int simt_recurrent_fw(int dtype, int state_dtype, const void* k, const void* v, const GateBuffers& gb,
                      const float* c_initial, const float* n_initial, void* c_states, float* n_states,
                      float* c_last, float* n_last, const ChunkwiseDims& d, cudaStream_t st);
int simt_parallel_fw(int dtype, int state_dtype, const void* q, const void* k, const void* v, const GateBuffers& gb,
                     const void* c_states, const float* n_states, void* h, float* n_out, const ChunkwiseDims& d,
                     cudaStream_t st);
int simt_recurrent_bw(int dtype, int state_dtype, const void* q, const void* dh, const GateBuffers& gb,
                      const float* dc_last, void* dc_states, float* dc_initial, const ChunkwiseDims& d,
                      cudaStream_t st);
int simt_parallel_bw(int dtype, int state_dtype, const void* q, const void* k, const void* v, const void* dh,
                     const GateBuffers& gb, const void* c_states, const void* dc_states, void* dq, void* dk, void* dv,
                     const ChunkwiseDims& d, cudaStream_t st);

// chunkwise_sm100.cu : tcgen05 + TMA kernels (bf16 / fp16, L = 128, head dims multiples of 8)
bool sm100_supported(int S, int DHQK, int DHHV, int L, int dtype);
bool sm100_sizes_ok(int B, int NH, int S, int DHQK, int DHHV);
// A launch may cover a sub-range of the B * NH independent (batch, head) units; all pointers stay those of the whole
// problem.  count < 0: every unit from `first` on.
struct UnitRange { int first = 0; int count = -1; };
int sm100_recurrent_fw(const void* k, const void* v, const GateBuffers& gb, const float* c_initial,
                       const float* n_initial, void* c_states, float* n_states, float* c_last, float* n_last,
                       const ChunkwiseDims& d, cudaStream_t st, UnitRange ur = UnitRange());
int sm100_parallel_fw(const void* q, const void* k, const void* v, const GateBuffers& gb, const void* c_states,
                      const float* n_states, void* h, float* n_out, const ChunkwiseDims& d, cudaStream_t st,
                      UnitRange ur = UnitRange());
int sm100_recurrent_bw(const void* q, const void* dh, const GateBuffers& gb, const float* dc_last, void* dc_states,
                       float* dc_initial, const ChunkwiseDims& d, cudaStream_t st, UnitRange ur = UnitRange());
int sm100_parallel_bw(const void* q, const void* k, const void* v, const void* dh, const GateBuffers& gb,
                      const void* c_states, const void* dc_states, void* dq, void* dk, void* dv, float* qdq_parts,
                      float* kdk_parts, const ChunkwiseDims& d, cudaStream_t st, UnitRange ur = UnitRange());
// number of CTAs the recurrence launches for the whole problem with 128-column state tiles, and SMs of the device
long sm100_recurrence_ctas(const ChunkwiseDims& d);
int sm100_sm_count();

// Forward of mlstm_b200_chunkwise_fw; `allow_split` = false keeps every launch on the caller's stream (no stream or
// event of the library is created or used).
int chunkwise_fw_body(const void* q, const void* k, const void* v, const void* i, const void* f,
                      const float* c_initial, const float* n_initial, const float* m_initial, void* h,
                      float* n_out, float* m_out, void* c_states, float* n_states, float* m_states,
                      float* c_last, float* n_last, float* m_last, void* workspace, size_t workspace_bytes,
                      int B, int NH, int S, int DHQK, int DHHV, int L, int dtype, int gate_dtype, int variant,
                      int impl, float eps, void* stream, bool allow_split);

int sm100_device_status(int reset, int* status);
int sm100_wait_expiry_selftest(unsigned limit, int code, cudaStream_t st);
// make the runtime load the forward kernels' code on the current device now (CUDA loads modules lazily, on first use)
int sm100_force_load();
int gates_force_load();

// step.cu
int launch_step(const void* q, const void* k, const void* v, const void* i, const void* f, const void* c,
                const void* n, const void* m, void* h, void* c_new, void* n_new, void* m_new, int B, int NH, int DHQK,
                int DHHV, int dtype, int gate_dtype, int state_dtype, float eps, cudaStream_t st);
int launch_step_sequence(const void* q, const void* k, const void* v, const void* i, const void* f, const float* c,
                         const float* n, const float* m, void* h, float* c_new, float* n_new, float* m_new, int B,
                         int NH, int T, int DHQK, int DHHV, int dtype, int gate_dtype, float eps, cudaStream_t st);

}  // namespace mlstm
