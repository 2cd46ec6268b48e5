// Shared helpers for the mLSTM sm_100a kernels: element-type conversion, math, launch checks.
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <math.h>
#include <stdint.h>

#include "../../include/mlstm_b200.h"

namespace mlstm {

// ---- element types ---------------------------------------------------------------------
__device__ __forceinline__ float to_f32(float x) { return x; }
__device__ __forceinline__ float to_f32(__nv_bfloat16 x) { return __bfloat162float(x); }
__device__ __forceinline__ float to_f32(__half x) { return __half2float(x); }

template <typename T> __device__ __forceinline__ T from_f32(float x);
template <> __device__ __forceinline__ float from_f32<float>(float x) { return x; }
template <> __device__ __forceinline__ __nv_bfloat16 from_f32<__nv_bfloat16>(float x) { return __float2bfloat16_rn(x); }
template <> __device__ __forceinline__ __half from_f32<__half>(float x) { return __float2half_rn(x); }

// ---- math ---------------------------------------------------------------------------------
// log(sigmoid(x)) without overflow, full-precision transcendental functions.
__device__ __forceinline__ float logsigmoid_f(float x) { return fminf(x, 0.f) - log1pf(expf(-fabsf(x))); }
__device__ __forceinline__ float sigmoid_f(float x) { return 1.f / (1.f + expf(-x)); }

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}

// ---- host side --------------------------------------------------------------------------
void set_last_cuda_error(cudaError_t e, const char* where);

#define MLSTM_CUDA_CHECK(expr)                         \
  do {                                                 \
    cudaError_t _e = (expr);                           \
    if (_e != cudaSuccess) {                           \
      ::mlstm::set_last_cuda_error(_e, #expr);         \
      return MLSTM_ERR_CUDA;                           \
    }                                                  \
  } while (0)

// every kernel launch of this library is counted (mlstm_b200_launch_count)
void note_launch();
#define MLSTM_LAUNCH_CHECK()                  \
  do {                                        \
    ::mlstm::note_launch();                   \
    MLSTM_CUDA_CHECK(cudaGetLastError());     \
  } while (0)

// Optional per-phase device timing (mlstm_b200_profile_*): when enabled, a pair of CUDA events
// brackets each phase on the launching stream.
enum Phase { PH_GATES = 0, PH_REC_FW, PH_PAR_FW, PH_REC_BW, PH_PAR_BW, PH_GATE_GRADS, PH_STEP, PH_COUNT };
struct PhaseScope {
  PhaseScope(int phase, cudaStream_t st);
  ~PhaseScope();
  int slot;
  cudaStream_t st;
  bool nvtx;
};

inline int ceil_div(int a, int b) { return (a + b - 1) / b; }
inline size_t align_up(size_t x, size_t a) { return (x + a - 1) / a * a; }
inline bool is_pow2(int x) { return x > 0 && (x & (x - 1)) == 0; }
inline size_t dtype_size(int dtype) { return dtype == MLSTM_F32 ? 4 : 2; }

// Problem description passed to every launcher.
// The last chunk may be ragged (S not a multiple of L; tcgen05 path only): NC = ceil(S / L) and the library's own
// per-token vectors are laid out with SP = NC * L slots per (batch, head), the slots past S holding neutral values
// (input gate switched off, nothing decays), so that the contraction kernels need no per-token bounds checks on
// them.  User-visible per-token arrays (i, f, n_out, m_out, dI, dF) keep S entries per (batch, head).
struct ChunkwiseDims {
  int B, NH, S, DHQK, DHHV, L, NC;
  int variant;  // MLSTM_EXP / MLSTM_SIG / MLSTM_SIG_NONORM
  float eps;
  float qk_scale;
  int SP;       // NC * L
  int dtype;    // element type of q, k, v, h and the gradients (MLSTM_F32 / MLSTM_BF16 / MLSTM_F16)
};
inline ChunkwiseDims make_dims(int B, int NH, int S, int DHQK, int DHHV, int L, int variant, float eps, int dtype) {
  const int NC = (S + L - 1) / L;
  return ChunkwiseDims{B, NH, S, DHQK, DHHV, L, NC, variant, eps, 1.0f / sqrtf((float)DHQK), NC * L, dtype};
}

// Per-token / per-chunk gate vectors produced by the gate pre-pass (all f32, device memory).
// Per-token arrays have SP slots per (batch, head) (see ChunkwiseDims).
struct GateBuffers {
  float* vecB;     // (BNH, S)  in-chunk inclusive cumsum of logsigmoid(f)
  float* iota;     // (BNH, S)  i, or logsigmoid(i) for the sigmoid input gate
  float* m_tok;    // (BNH, S)  combined max state per token (0 for the sigmoid gate)
  float* abar;     // (BNH, S)  exp(a_j - m_{k+1})
  float* bbar;     // (BNH, S)  exp(b_i + m_k - m_i)
  float* gbar;     // (BNH, NC) exp(g_k + m_k - m_{k+1})
  float* inv_den;  // (BNH, S)  backward only: 1 / (n_out + eps) (1 when there is no normaliser)
  float* scratch;  // (BNH, 2*NC) per-chunk g and max_j a_j
};

}  // namespace mlstm
