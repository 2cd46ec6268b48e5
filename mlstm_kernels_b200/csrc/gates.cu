// Gate pre-pass and gate-gradient kernels (scalar work per token; HBM traffic is negligible).
//
// Pre-pass: from the raw gate logits i, f produce every per-token and per-chunk scalar the
// contraction kernels need, including the serial max-state recursion over chunks, which is
// evaluated as a block-wide scan over (max,+) affine maps.
// Follows mlstm_kernels/torch/chunkwise/triton_xl_chunk/chunkwise_gates.py:15-65 (vecB, vecA),
// mlstm_kernels/triton/chunkwise/xl_chunk/fw_kernel_recurrent.py:150-176 (m recursion) and
// mlstm_kernels/torch/chunkwise/native/fw.py:178-195 (per-token max state).
#include <algorithm>

#include "common.cuh"
#include "launch.cuh"

namespace mlstm {

constexpr int kGateThreads = 256;

// The pre-pass runs as three launches so that the per-chunk work (1 and 3) spreads over the whole GPU and only
// the scan over chunks (2) is serial per (batch, head):
//   gates_chunk_kernel  b_j, a_j, g_k, max_j a_j           one warp per chunk
//   gates_scan_kernel   m_k, gbar_k, total G               one CTA per (batch, head)
//   gates_token_kernel  m_i, abar_j, bbar_i, 1/(den+eps)   one warp per chunk
template <typename T>
__global__ void __launch_bounds__(kGateThreads)
gates_chunk_kernel(const T* __restrict__ vecI, const T* __restrict__ vecF, GateBuffers gb, int S, int SP, int L,
                   int NC, int variant) {
  // 1-D grid (no 65535 limit on batch x heads): the chunk groups of one (batch, head) next to each other
  const int ngrp = (NC + kGateThreads / 32 - 1) / (kGateThreads / 32);
  const int bh = blockIdx.x / ngrp;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int k = (blockIdx.x % ngrp) * (kGateThreads / 32) + warp;
  if (k >= NC) return;
  const bool siging = variant != MLSTM_EXP;
  float* g_arr = gb.scratch + (size_t)bh * 2 * NC;
  float* amax_arr = g_arr + NC;
  // inputs have S tokens per (batch, head), the gate vectors SP = NC * L slots; slots past the sequence end are
  // filled with neutral values: log forget gate 0 (nothing decays), input gate -inf (contributes nothing)
  const size_t base_in = (size_t)bh * S + (size_t)k * L;
  const size_t base = (size_t)bh * SP + (size_t)k * L;
  const int valid = min(L, S - k * L);
  float carry = 0.f;
  for (int j0 = 0; j0 < L; j0 += 32) {
    const int j = j0 + lane;
    float x = (j < valid) ? logsigmoid_f(to_f32(vecF[base_in + j])) : 0.f;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      float y = __shfl_up_sync(0xffffffffu, x, o);
      if (lane >= o) x += y;
    }
    x += carry;
    if (j < L) gb.vecB[base + j] = x;
    carry = __shfl_sync(0xffffffffu, x, 31);
  }
  const float g = carry;
  // a_j = sum_{t>j} lf_t + iota_j as a reverse scan that never includes position j
  float suffix = 0.f, amax = -INFINITY;
  for (int j0 = ((L - 1) / 32) * 32; j0 >= 0; j0 -= 32) {
    const int j = j0 + lane;
    float x = (j < valid) ? logsigmoid_f(to_f32(vecF[base_in + j])) : 0.f;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      float y = __shfl_down_sync(0xffffffffu, x, o);
      if (lane + o < 32) x += y;
    }
    float excl = __shfl_down_sync(0xffffffffu, x, 1);
    if (lane == 31) excl = 0.f;
    excl += suffix;
    suffix += __shfl_sync(0xffffffffu, x, 0);
    if (j < L) {
      float iota = -INFINITY;
      if (j < valid) {
        const float iv = to_f32(vecI[base_in + j]);
        iota = siging ? logsigmoid_f(iv) : iv;
      }
      const float a = excl + iota;
      gb.iota[base + j] = iota;
      gb.abar[base + j] = a;  // finalised by gates_token_kernel
      amax = fmaxf(amax, a);
    }
  }
  amax = warp_max(amax);
  if (lane == 0) { g_arr[k] = g; amax_arr[k] = amax; }
}

// m_{k+1} = max(g_k + m_k, amax_k) as a block scan over the maps x -> max(x + G, A)
__global__ void __launch_bounds__(kGateThreads)
gates_scan_kernel(const float* __restrict__ m_initial, GateBuffers gb, float* __restrict__ m_states, int NC,
                  int variant, float m_default, float* __restrict__ g_sum) {
  __shared__ float sG[kGateThreads], sA[kGateThreads], sMin[kGateThreads];
  const int bh = blockIdx.x, t = threadIdx.x;
  const bool siging = variant != MLSTM_EXP;
  const float* g_arr = gb.scratch + (size_t)bh * 2 * NC;
  const float* amax_arr = g_arr + NC;
  const int seg = (NC + kGateThreads - 1) / kGateThreads;
  const int k0 = min(NC, t * seg), k1 = min(NC, (t + 1) * seg);
  float* ms = m_states + (size_t)bh * (NC + 1);
  float G = 0.f, A = -INFINITY;
  for (int k = k0; k < k1; ++k) { A = fmaxf(A + g_arr[k], amax_arr[k]); G += g_arr[k]; }
  sG[t] = G; sA[t] = A;
  __syncthreads();
  if (t == 0) {
    float m = m_initial ? m_initial[bh] : m_default;
    float Gt = 0.f;
    for (int u = 0; u < kGateThreads; ++u) { sMin[u] = m; m = fmaxf(m + sG[u], sA[u]); Gt += sG[u]; }
    if (g_sum != nullptr) g_sum[bh] = Gt;   // total log forget gate of the sequence (for chaining segments)
  }
  __syncthreads();
  if (!siging) {
    float m = sMin[t];
    for (int k = k0; k < k1; ++k) {
      ms[k] = m;
      const float mn = fmaxf(g_arr[k] + m, amax_arr[k]);
      gb.gbar[(size_t)bh * NC + k] = expf(g_arr[k] + m - mn);
      m = mn;
      if (k == NC - 1) ms[NC] = m;
    }
  } else {
    for (int k = k0; k < k1; ++k) {
      ms[k] = 0.f;
      gb.gbar[(size_t)bh * NC + k] = expf(g_arr[k]);
      if (k == NC - 1) ms[NC] = 0.f;
    }
  }
}

__global__ void __launch_bounds__(kGateThreads)
gates_token_kernel(const float* __restrict__ n_out, float* __restrict__ m_out, GateBuffers gb,
                   const float* __restrict__ m_states, int S, int SP, int L, int NC, int variant, float eps) {
  // 1-D grid (no 65535 limit on batch x heads): the chunk groups of one (batch, head) next to each other
  const int ngrp = (NC + kGateThreads / 32 - 1) / (kGateThreads / 32);
  const int bh = blockIdx.x / ngrp;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int k = (blockIdx.x % ngrp) * (kGateThreads / 32) + warp;
  if (k >= NC) return;
  const bool siging = variant != MLSTM_EXP;
  const size_t base_in = (size_t)bh * S + (size_t)k * L;
  const size_t base = (size_t)bh * SP + (size_t)k * L;
  const int valid = min(L, S - k * L);
  const float m_prev = m_states[(size_t)bh * (NC + 1) + k];
  const float m_next = m_states[(size_t)bh * (NC + 1) + k + 1];
  float carry = -INFINITY;
  for (int j0 = 0; j0 < L; j0 += 32) {
    const int j = j0 + lane;
    float b = 0.f, x = -INFINITY;
    if (j < L) { b = gb.vecB[base + j]; x = gb.iota[base + j] - b; }
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      float y = __shfl_up_sync(0xffffffffu, x, o);
      if (lane >= o) x = fmaxf(x, y);
    }
    x = fmaxf(x, carry);
    carry = __shfl_sync(0xffffffffu, x, 31);
    if (j < L) {
      float m_i, bbar, abar;
      const float a = gb.abar[base + j];
      if (siging) {
        m_i = 0.f; bbar = expf(b); abar = expf(a);
      } else {
        m_i = fmaxf(b + m_prev, b + x);
        bbar = expf(b + m_prev - m_i);
        abar = expf(a - m_next);
      }
      const bool pad = j >= valid;     // slot past the sequence end: finite max state, every factor zero
      gb.m_tok[base + j] = m_i;
      gb.bbar[base + j] = pad ? 0.f : bbar;
      gb.abar[base + j] = pad ? 0.f : abar;
      if (m_out != nullptr && !pad) m_out[base_in + j] = m_i;
      if (gb.inv_den) {
        gb.inv_den[base + j] = pad ? 0.f
                               : ((variant == MLSTM_SIG_NONORM || n_out == nullptr) ? 1.f : 1.f / (n_out[base_in + j] + eps));
      }
    }
  }
}

// Per-token reductions for the gate gradients:
//   qdq_t = sum_d q dq,  kdk_t = sum_d k dk
// mlstm_kernels/torch/chunkwise/triton_xl_chunk/chunkwise_gates.py:68-95. One warp per token.
template <typename T>
__global__ void __launch_bounds__(256)
gate_grad_rows_kernel(const T* __restrict__ q, const T* __restrict__ k, const T* __restrict__ dq,
                      const T* __restrict__ dk, float* __restrict__ acc, float* __restrict__ kdk,
                      size_t ntok, int DHQK) {
  const size_t tok = (size_t)blockIdx.x * 8 + (threadIdx.x >> 5);
  if (tok >= ntok) return;
  const int lane = threadIdx.x & 31;
  const size_t base = tok * DHQK;
  float a = 0.f, b = 0.f;
  for (int d = lane; d < DHQK; d += 32) {
    a += to_f32(q[base + d]) * to_f32(dq[base + d]);
    b += to_f32(k[base + d]) * to_f32(dk[base + d]);
  }
  a = warp_sum(a); b = warp_sum(b);
  if (lane == 0) { acc[tok] = a; kdk[tok] = b; }
}

// deltaF_t = sigmoid(-f_t) * sum_{t' >= t over the whole sequence} (qdq_t' - kdk_t') ; deltaI_t = kdk_t (* sigmoid(-i_t)).
// qdq / kdk may arrive as `nparts` partial sums (one per 128-wide head-dim tile), `part_stride` floats apart;
// they are added in a fixed order, so the result does not depend on scheduling.
// One CTA per (batch, head); each thread owns a contiguous token range, block scan over the range sums.
//
// Anchors (tcgen05 path).  q.dq and k.dk nearly cancel, and what is left of their rounding errors (bf16 states and
// operands) adds up along the reverse sum like a random walk: its error grows with the square root of the sequence
// length.  At a chunk boundary the exact value of the sum is known in closed form: with C_k the state before chunk k
// and dC_k its gradient,  sum over all tokens t' >= k L of (q.dq - k.dk) = <C_k, dC_k> - <C_NC, dC_NC>
// (the per-chunk totals telescope: <C_k, dP_k> - <P_k, dC_{k+1}> = <C_k, dC_k> - <C_{k+1}, dC_{k+1}> for
// C_{k+1} = g C_k + P_k, dC_k = g dC_{k+1} + dP_k).  `anchors` holds those inner products for every
// `anchor_tokens`-th token position (state_dot_kernel); the running sum of a token is then taken from the next anchor
// instead of from the end of the sequence, which bounds the walk to one anchor interval (gate_grad_anchored_kernel).
// gate_grad_scan_kernel is the plain form (portable path: f32 states, no anchors).
constexpr int kScanThreads = 1024;
template <typename T>
__global__ void __launch_bounds__(kScanThreads)
gate_grad_scan_kernel(const T* __restrict__ vecI, const T* __restrict__ vecF, const float* __restrict__ qdq,
                      const float* __restrict__ kdk, float* __restrict__ dI, float* __restrict__ dF,
                      int S, int SP, int variant, int nparts, size_t part_stride) {
  __shared__ float s_part[kScanThreads];
  const int bh = blockIdx.x, t = threadIdx.x;
  const size_t base = (size_t)bh * S;      // gate logits and outputs: S tokens per (batch, head)
  const size_t pbase = (size_t)bh * SP;    // row sums: SP slots per (batch, head)
  const int seg = (S + kScanThreads - 1) / kScanThreads;
  const int s0 = min(S, t * seg), s1 = min(S, (t + 1) * seg);
  auto parts = [&](const float* src, size_t idx) {
    float t = 0.f;
    for (int pp = 0; pp < nparts; ++pp) t += src[pp * part_stride + idx];
    return t;
  };
  float sum = 0.f;
  for (int s = s0; s < s1; ++s) sum += parts(qdq, pbase + s) - parts(kdk, pbase + s);
  s_part[t] = sum;
  __syncthreads();
  // suffix sums over threads (exclusive): sum of the ranges to the right
  for (int o = 1; o < kScanThreads; o <<= 1) {
    float y = (t + o < kScanThreads) ? s_part[t + o] : 0.f;
    __syncthreads();
    s_part[t] += y;
    __syncthreads();
  }
  float run = (t + 1 < kScanThreads) ? s_part[t + 1] : 0.f;
  for (int s = s1 - 1; s >= s0; --s) {
    float di = parts(kdk, pbase + s);
    run += parts(qdq, pbase + s) - di;
    dF[base + s] = run * sigmoid_f(-to_f32(vecF[base + s]));
    if (variant != MLSTM_EXP) di *= sigmoid_f(-to_f32(vecI[base + s]));
    dI[base + s] = di;
  }
}

// The anchored form.  Between two anchors the running sum needs nothing from outside the interval: for a token t
// with next anchor position p,  sum_{t' >= t} = sum_{t <= t' < p} (qdq - kdk)  +  anchors[p] - anchors[end]
// (the last interval ends at the end of the sequence, where both anchor terms vanish).  So every interval of
// `anchor_tokens` tokens is an independent CTA: grid (intervals, batch x heads), one token per thread, the suffix
// sum inside the interval by warp shuffles in a fixed order.
constexpr int kAnchorThreads = 512;
template <typename T>
__global__ void __launch_bounds__(kAnchorThreads)
gate_grad_anchored_kernel(const T* __restrict__ vecI, const T* __restrict__ vecF, const float* __restrict__ qdq,
                          const float* __restrict__ kdk, float* __restrict__ dI, float* __restrict__ dF, int S,
                          int SP, int variant, int nparts, size_t part_stride,
                          const float* __restrict__ anchors, int n_anchors) {
  __shared__ float s_warp[kAnchorThreads / 32];
  const int nint = (S + kAnchorThreads - 1) / kAnchorThreads;   // 1-D grid: intervals of one (batch, head) adjacent
  const int a = blockIdx.x % nint, bh = blockIdx.x / nint, t = threadIdx.x, lane = t & 31, warp = t >> 5;
  const int s = a * kAnchorThreads + t;
  const bool live = s < S;
  float qd = 0.f, kd = 0.f;
  if (live) {
    const size_t idx = (size_t)bh * SP + s;
    for (int pp = 0; pp < nparts; ++pp) { qd += qdq[pp * part_stride + idx]; kd += kdk[pp * part_stride + idx]; }
  }
  // inclusive suffix sum over the interval: inside the warp, then over the warps to the right
  float x = qd - kd;
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    const float y = __shfl_down_sync(0xffffffffu, x, o);
    if (lane + o < 32) x += y;
  }
  if (lane == 0) s_warp[warp] = x;
  __syncthreads();
  float right = 0.f;
  for (int w = kAnchorThreads / 32 - 1; w > warp; --w) right += s_warp[w];
  float total = x + right;
  if (a + 1 < n_anchors - 1) {   // the interval ends at an interior anchor
    const float* anc = anchors + (size_t)bh * n_anchors;
    total += anc[a + 1] - anc[n_anchors - 1];
  }
  if (live) {
    const size_t o = (size_t)bh * S + s;
    dF[o] = total * sigmoid_f(-to_f32(vecF[o]));
    dI[o] = (variant != MLSTM_EXP) ? kd * sigmoid_f(-to_f32(vecI[o])) : kd;
  }
}

// anchors[bh][a] = <C_k, dC_k> over the whole DHQK x DHHV state, k = min(a * every, NC), a = 1 .. n_anchors - 1
// (a = 0 is never read).  One CTA per (anchor, batch x head); the partial sums are added in a fixed order.
template <typename TS>
__global__ void __launch_bounds__(256)
state_dot_kernel(const TS* __restrict__ c_states, const TS* __restrict__ dc_states,
                 float* __restrict__ anchors, int NC, int every, int n_anchors, size_t state_elems) {
  __shared__ float s_w[8];
  const int bh = blockIdx.x / (n_anchors - 1), a = blockIdx.x % (n_anchors - 1) + 1;   // 1-D grid
  const int k = min(a * every, NC);
  const size_t off = ((size_t)bh * (NC + 1) + k) * state_elems;
  const uint4* pc = reinterpret_cast<const uint4*>(c_states + off);
  const uint4* pd = reinterpret_cast<const uint4*>(dc_states + off);
  float acc[4] = {0.f, 0.f, 0.f, 0.f};
  for (size_t idx = threadIdx.x; idx < state_elems / 8; idx += 256) {
    const uint4 x = __ldcs(pc + idx), y = __ldcs(pd + idx);
    const uint32_t xw[4] = {x.x, x.y, x.z, x.w}, yw[4] = {y.x, y.y, y.z, y.w};
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const TS* xa = reinterpret_cast<const TS*>(&xw[e]);
      const TS* ya = reinterpret_cast<const TS*>(&yw[e]);
      acc[e] = fmaf(to_f32(xa[0]), to_f32(ya[0]), acc[e]);
      acc[e] = fmaf(to_f32(xa[1]), to_f32(ya[1]), acc[e]);
    }
  }
  float v = warp_sum((acc[0] + acc[1]) + (acc[2] + acc[3]));
  if ((threadIdx.x & 31) == 0) s_w[threadIdx.x >> 5] = v;
  __syncthreads();
  if (threadIdx.x == 0) {
    float tot = 0.f;
    for (int w = 0; w < 8; ++w) tot += s_w[w];
    anchors[(size_t)bh * n_anchors + a] = tot;
  }
}

// ---- launchers ----------------------------------------------------------------------------------
template <typename T>
int launch_gates_t(const void* i, const void* f, const float* m_initial, const float* n_out, float* m_out,
                   const GateBuffers& gb, float* m_states, const ChunkwiseDims& d, cudaStream_t st, float m_default,
                   float* g_sum) {
  PhaseScope ps(PH_GATES, st);
  const unsigned grid = (unsigned)ceil_div(d.NC, kGateThreads / 32) * (unsigned)(d.B * d.NH);
  gates_chunk_kernel<T><<<grid, kGateThreads, 0, st>>>((const T*)i, (const T*)f, gb, d.S, d.SP, d.L, d.NC, d.variant);
  MLSTM_LAUNCH_CHECK();
  gates_scan_kernel<<<d.B * d.NH, kGateThreads, 0, st>>>(m_initial, gb, m_states, d.NC, d.variant, m_default, g_sum);
  MLSTM_LAUNCH_CHECK();
  gates_token_kernel<<<grid, kGateThreads, 0, st>>>(n_out, m_out, gb, m_states, d.S, d.SP, d.L, d.NC, d.variant, d.eps);
  MLSTM_LAUNCH_CHECK();
  return MLSTM_OK;
}

int launch_gates(int dtype, const void* i, const void* f, const float* m_initial, const float* n_out, float* m_out,
                 const GateBuffers& gb, float* m_states, const ChunkwiseDims& d, cudaStream_t st, float m_default,
                 float* g_sum) {
  switch (dtype) {
    case MLSTM_F32: return launch_gates_t<float>(i, f, m_initial, n_out, m_out, gb, m_states, d, st, m_default, g_sum);
    case MLSTM_BF16: return launch_gates_t<__nv_bfloat16>(i, f, m_initial, n_out, m_out, gb, m_states, d, st, m_default, g_sum);
    case MLSTM_F16: return launch_gates_t<__half>(i, f, m_initial, n_out, m_out, gb, m_states, d, st, m_default, g_sum);
  }
  return MLSTM_ERR_DTYPE;
}

int gates_force_load() {
  cudaFuncAttributes a;
  MLSTM_CUDA_CHECK(cudaFuncGetAttributes(&a, gates_chunk_kernel<float>));
  MLSTM_CUDA_CHECK(cudaFuncGetAttributes(&a, gates_chunk_kernel<__nv_bfloat16>));
  MLSTM_CUDA_CHECK(cudaFuncGetAttributes(&a, gates_chunk_kernel<__half>));
  MLSTM_CUDA_CHECK(cudaFuncGetAttributes(&a, gates_scan_kernel));
  MLSTM_CUDA_CHECK(cudaFuncGetAttributes(&a, gates_token_kernel));
  return MLSTM_OK;
}

template <typename T>
int launch_gate_grad_rows_t(const void* q, const void* k, const void* dq, const void* dk, float* acc, float* kdk,
                            const ChunkwiseDims& d, cudaStream_t st) {
  const size_t ntok = (size_t)d.B * d.NH * d.S;
  gate_grad_rows_kernel<T><<<(unsigned)((ntok + 7) / 8), 256, 0, st>>>((const T*)q, (const T*)k, (const T*)dq,
                                                                        (const T*)dk, acc, kdk, ntok, d.DHQK);
  MLSTM_LAUNCH_CHECK();
  return MLSTM_OK;
}



int launch_gate_grads(int dtype, int gate_dtype, const void* q, const void* k, const void* dq, const void* dk,
                      const void* i, const void* f, float* acc, float* kdk, float* dI, float* dF,
                      const ChunkwiseDims& d, cudaStream_t st) {
  PhaseScope ps(PH_GATE_GRADS, st);
  int rc = MLSTM_ERR_DTYPE;
  switch (dtype) {
    case MLSTM_F32: rc = launch_gate_grad_rows_t<float>(q, k, dq, dk, acc, kdk, d, st); break;
    case MLSTM_BF16: rc = launch_gate_grad_rows_t<__nv_bfloat16>(q, k, dq, dk, acc, kdk, d, st); break;
    case MLSTM_F16: rc = launch_gate_grad_rows_t<__half>(q, k, dq, dk, acc, kdk, d, st); break;
  }
  if (rc != MLSTM_OK) return rc;
  return launch_gate_grad_scan(gate_dtype, i, f, acc, kdk, 1, dI, dF, d, st, nullptr, 0, 1);
}

// Joins the state a sequence segment produced from the EMPTY state (C = 0, n = 0, m = -inf) onto the state that
// enters the segment:  m_out = max(G + m_in, m_loc),  X_out = exp(G + m_in - m_out) X_in + exp(m_loc - m_out) X_loc
// for X in {C, n}; G = total log forget gate of the segment.  Same recursion as the per-chunk update
// (mlstm_kernels/triton/chunkwise/xl_chunk/fw_kernel_recurrent.py:175-196) applied to a whole segment.
__global__ void __launch_bounds__(256)
state_combine_kernel(const float* __restrict__ c_in, const float* __restrict__ n_in, const float* __restrict__ m_in,
                     const float* __restrict__ c_loc, const float* __restrict__ n_loc, const float* __restrict__ m_loc,
                     const float* __restrict__ g_total, float* __restrict__ c_out, float* __restrict__ n_out,
                     float* __restrict__ m_out, int DHQK, int DHHV, int variant, int nblk) {
  const int bh = blockIdx.x / nblk, blk = blockIdx.x % nblk;   // 1-D grid: nblk CTAs per (batch, head)
  float a, b, mo = 0.f;
  if (variant == MLSTM_EXP) {
    const float mi = m_in ? m_in[bh] : 0.f, ml = m_loc[bh], G = g_total[bh];
    mo = fmaxf(G + mi, ml);
    a = expf(G + mi - mo);
    b = expf(ml - mo);
  } else {
    a = expf(g_total[bh]);
    b = 1.f;
  }
  const size_t nC = (size_t)DHQK * DHHV;
  for (size_t e = (size_t)blk * blockDim.x + threadIdx.x; e < nC; e += (size_t)nblk * blockDim.x) {
    const size_t idx = (size_t)bh * nC + e;
    c_out[idx] = a * (c_in ? c_in[idx] : 0.f) + b * c_loc[idx];
    if (e < (size_t)DHQK && n_out != nullptr) {
      const size_t ni = (size_t)bh * DHQK + e;
      n_out[ni] = a * (n_in ? n_in[ni] : 0.f) + b * n_loc[ni];
    }
  }
  if (blk == 0 && threadIdx.x == 0 && m_out != nullptr) m_out[bh] = mo;
}

int launch_state_combine(const float* c_in, const float* n_in, const float* m_in, const float* c_loc,
                         const float* n_loc, const float* m_loc, const float* g_total, float* c_out, float* n_out,
                         float* m_out, int BNH, int DHQK, int DHHV, int variant, cudaStream_t st) {
  const size_t nC = (size_t)DHQK * DHHV;
  const int nblk = (int)std::min<size_t>((nC + 255) / 256, 64);
  state_combine_kernel<<<(unsigned)nblk * (unsigned)BNH, 256, 0, st>>>(c_in, n_in, m_in, c_loc, n_loc, m_loc, g_total,
                                                                      c_out, n_out, m_out, DHQK, DHHV, variant, nblk);
  MLSTM_LAUNCH_CHECK();
  return MLSTM_OK;
}

// inv_den_t = 1 / (n_out_t + eps), or 1 where the variant has no normaliser; 0 in the slots past the sequence end
// (n_out has S entries per (batch, head), inv_den SP slots)
__global__ void __launch_bounds__(256)
inv_den_kernel(const float* __restrict__ n_out, float* __restrict__ inv_den, size_t nslots, int S, int SP, int variant,
               float eps) {
  const size_t t = (size_t)blockIdx.x * 256 + threadIdx.x;
  if (t >= nslots) return;
  const size_t bh = t / SP;
  const int s = (int)(t - bh * SP);
  float v = 0.f;
  if (s < S) v = (variant == MLSTM_SIG_NONORM || n_out == nullptr) ? 1.f : 1.f / (n_out[bh * S + s] + eps);
  inv_den[t] = v;
}

int launch_inv_den(const float* n_out, float* inv_den, const ChunkwiseDims& d, cudaStream_t st) {
  PhaseScope ps(PH_GATES, st);
  const size_t nslots = (size_t)d.B * d.NH * d.SP;
  inv_den_kernel<<<(unsigned)((nslots + 255) / 256), 256, 0, st>>>(n_out, inv_den, nslots, d.S, d.SP, d.variant, d.eps);
  MLSTM_LAUNCH_CHECK();
  return MLSTM_OK;
}

// Scan-only entry: the row sums were already produced (in f32, before rounding) by the backward kernels.
// With `anchors` (see above) the sum restarts from an exact value every `anchor_tokens` tokens and the intervals run
// as independent CTAs; without, one CTA per (batch, head) scans the whole sequence.
template <typename T>
static int gate_grad_scan_t(const void* i, const void* f, const float* qdq, const float* kdk, int nparts, float* dI,
                            float* dF, const ChunkwiseDims& d, cudaStream_t st, const float* anchors, int n_anchors,
                            int anchor_tokens) {
  const size_t stride = (size_t)d.B * d.NH * d.SP;
  if (anchors != nullptr && anchor_tokens == kAnchorThreads) {
    const unsigned grid = (unsigned)ceil_div(d.S, kAnchorThreads) * (unsigned)(d.B * d.NH);
    gate_grad_anchored_kernel<T><<<grid, kAnchorThreads, 0, st>>>((const T*)i, (const T*)f, qdq, kdk, dI, dF, d.S, d.SP,
                                                                  d.variant, nparts, stride, anchors, n_anchors);
  } else {
    gate_grad_scan_kernel<T><<<d.B * d.NH, kScanThreads, 0, st>>>((const T*)i, (const T*)f, qdq, kdk, dI, dF, d.S, d.SP,
                                                                  d.variant, nparts, stride);
  }
  MLSTM_LAUNCH_CHECK();
  return MLSTM_OK;
}

int launch_gate_grad_scan(int dtype, const void* i, const void* f, const float* qdq, const float* kdk, int nparts,
                          float* dI, float* dF, const ChunkwiseDims& d, cudaStream_t st, const float* anchors,
                          int n_anchors, int anchor_tokens) {
  switch (dtype) {
    case MLSTM_F32: return gate_grad_scan_t<float>(i, f, qdq, kdk, nparts, dI, dF, d, st, anchors, n_anchors, anchor_tokens);
    case MLSTM_BF16: return gate_grad_scan_t<__nv_bfloat16>(i, f, qdq, kdk, nparts, dI, dF, d, st, anchors, n_anchors, anchor_tokens);
    case MLSTM_F16: return gate_grad_scan_t<__half>(i, f, qdq, kdk, nparts, dI, dF, d, st, anchors, n_anchors, anchor_tokens);
  }
  return MLSTM_ERR_DTYPE;
}

// <C_k, dC_k> at every `every`-th chunk boundary and at the end (16-bit states of the tcgen05 path).
int launch_state_dot(const void* c_states, const void* dc_states, float* anchors, int every, int n_anchors,
                     const ChunkwiseDims& d, cudaStream_t st) {
  if (n_anchors < 2) return MLSTM_OK;
  const unsigned grid = (unsigned)(n_anchors - 1) * (unsigned)(d.B * d.NH);
  if (d.dtype == MLSTM_F16)
    state_dot_kernel<__half><<<grid, 256, 0, st>>>((const __half*)c_states, (const __half*)dc_states, anchors, d.NC,
                                                   every, n_anchors, (size_t)d.DHQK * d.DHHV);
  else
    state_dot_kernel<__nv_bfloat16><<<grid, 256, 0, st>>>((const __nv_bfloat16*)c_states, (const __nv_bfloat16*)dc_states,
                                                          anchors, d.NC, every, n_anchors, (size_t)d.DHQK * d.DHHV);
  MLSTM_LAUNCH_CHECK();
  return MLSTM_OK;
}

}  // namespace mlstm
