// Portable CUDA-core implementation of the chunkwise mLSTM kernels (any chunk size >= 16, any head
// dimension, f32 / bf16 / f16 inputs, exact f32 arithmetic).  It covers the shapes the tcgen05 path
// does not (small chunks, odd head dims, f32 inputs) and is the on-device cross-check for it.
//
//   rec_kernel  : inter-chunk recurrence, forward (C_k, n_k) and backward (deltaC_k)
//                 mlstm_kernels/triton/chunkwise/xl_chunk/fw_kernel_recurrent.py:14-230,
//                 bw_kernel_recurrent.py:15-181
//   par_kernel  : intra-chunk gated products + inter-chunk contribution for H, deltaV, deltaK, deltaQ
//                 fw_kernel_parallel.py:14-289, bw_kernel_parallel_dV.py, _dK.py, _dQ.py
#include "common.cuh"
#include "launch.cuh"

namespace mlstm {

constexpr int TILE = 64;   // output tile edge per CTA
constexpr int KSL = 32;    // contraction slice staged in shared memory
constexpr int NTHR = 256;  // 16 x 16 threads, 4 x 4 outputs each

// =====================================================================================================
// Inter-chunk recurrence.  state <- gbar * state + (left * lscale * lmul)^T (right * rscale)
//   forward : left = K, lscale = abar, right = V;  also n <- gbar n + sum_j abar_j k_j
//   backward: left = Q, lscale = bbar, lmul = qk_scale, right = deltaH, rscale = 1/(den+eps); chunks reversed
// grid (ceil(DHHV/64) * B*NH, ceil(DHQK/64))
// =====================================================================================================
template <typename T, typename TS, bool BWD>
__global__ void __launch_bounds__(NTHR)
rec_kernel(const T* __restrict__ left, const T* __restrict__ right, const float* __restrict__ lscale, float lmul,
           const float* __restrict__ rscale, const float* __restrict__ gbar, const float* __restrict__ c_init,
           const float* __restrict__ n_init, TS* __restrict__ c_states, float* __restrict__ n_states,
           float* __restrict__ c_final, float* __restrict__ n_final, int S, int L, int NC, int DHQK, int DHHV) {
  __shared__ float Ls[KSL][TILE + 1];
  __shared__ float Rs[KSL][TILE + 1];
  const int tid = threadIdx.x, tx = tid & 15, ty = tid >> 4;
  // grid (column tiles x batch x heads, row tiles): batch x heads sits in x, which has no 65535 limit
  const int n_et = (DHHV + TILE - 1) / TILE, et = blockIdx.x % n_et;
  const int e0 = et * TILE, d0 = blockIdx.y * TILE, bh = blockIdx.x / n_et;
  const bool do_n = (!BWD) && (et == 0) && (n_states != nullptr || n_final != nullptr);

  float C[4][4];
#pragma unroll
  for (int a = 0; a < 4; ++a)
#pragma unroll
    for (int b = 0; b < 4; ++b) {
      const int d = d0 + ty * 4 + a, e = e0 + tx * 4 + b;
      C[a][b] = (c_init && d < DHQK && e < DHHV) ? c_init[((size_t)bh * DHQK + d) * DHHV + e] : 0.f;
    }
  float nval = 0.f;
  if (do_n && tid < TILE && d0 + tid < DHQK && n_init) nval = n_init[(size_t)bh * DHQK + d0 + tid];

  auto store_state = [&](int slot) {
    if (c_states != nullptr) {
      TS* cs = c_states + ((size_t)bh * (NC + 1) + slot) * DHQK * DHHV;
#pragma unroll
      for (int a = 0; a < 4; ++a)
#pragma unroll
        for (int b = 0; b < 4; ++b) {
          const int d = d0 + ty * 4 + a, e = e0 + tx * 4 + b;
          if (d < DHQK && e < DHHV) cs[(size_t)d * DHHV + e] = from_f32<TS>(C[a][b]);
        }
    }
    if (do_n && n_states != nullptr && tid < TILE && d0 + tid < DHQK) n_states[((size_t)bh * (NC + 1) + slot) * DHQK + d0 + tid] = nval;
  };

  for (int s = 0; s < NC; ++s) {
    const int slot = BWD ? NC - s : s;
    const int ck = BWD ? NC - 1 - s : s;
    store_state(slot);
    const size_t tok0 = (size_t)bh * S + (size_t)ck * L;
    float acc[4][4] = {};
    float nacc = 0.f;
    for (int r0 = 0; r0 < L; r0 += KSL) {
      for (int idx = tid; idx < KSL * TILE; idx += NTHR) {
        const int r = idx / TILE, c = idx % TILE;
        const int row = r0 + r;
        float lv = 0.f, rv = 0.f;
        if (row < L) {
          const size_t tok = tok0 + row;
          if (d0 + c < DHQK) lv = to_f32(left[tok * DHQK + d0 + c]) * (lscale[tok] * lmul);
          if (e0 + c < DHHV) rv = to_f32(right[tok * DHHV + e0 + c]) * (rscale ? rscale[tok] : 1.f);
        }
        Ls[r][c] = lv;
        Rs[r][c] = rv;
      }
      __syncthreads();
#pragma unroll 8
      for (int r = 0; r < KSL; ++r) {
        float a4[4], b4[4];
#pragma unroll
        for (int a = 0; a < 4; ++a) a4[a] = Ls[r][ty * 4 + a];
#pragma unroll
        for (int b = 0; b < 4; ++b) b4[b] = Rs[r][tx * 4 + b];
#pragma unroll
        for (int a = 0; a < 4; ++a)
#pragma unroll
          for (int b = 0; b < 4; ++b) acc[a][b] = fmaf(a4[a], b4[b], acc[a][b]);
      }
      if (do_n && tid < TILE) {
#pragma unroll 8
        for (int r = 0; r < KSL; ++r) nacc += Ls[r][tid];
      }
      __syncthreads();
    }
    const float g = gbar[(size_t)bh * NC + ck];
#pragma unroll
    for (int a = 0; a < 4; ++a)
#pragma unroll
      for (int b = 0; b < 4; ++b) C[a][b] = fmaf(g, C[a][b], acc[a][b]);
    nval = fmaf(g, nval, nacc);
  }
  store_state(BWD ? 0 : NC);
  if (c_final) {
#pragma unroll
    for (int a = 0; a < 4; ++a)
#pragma unroll
      for (int b = 0; b < 4; ++b) {
        const int d = d0 + ty * 4 + a, e = e0 + tx * 4 + b;
        if (d < DHQK && e < DHHV) c_final[((size_t)bh * DHQK + d) * DHHV + e] = C[a][b];
      }
  }
  if (do_n && n_final && tid < TILE && d0 + tid < DHQK) n_final[(size_t)bh * DHQK + d0 + tid] = nval;
}

// =====================================================================================================
// Intra-chunk kernel, four modes.  For the output tile rows r (tokens of one chunk) and columns o:
//   out[r,o] = sum_c P[r,c] X[c,o] + rowscale_r * sum_a A[r,a] Bm[a,o]
//   P[r,c]   = qk_scale * (U[r] . W[c]) * D(i,j),  D(i,j) = exp((b_i - b_j) + iota_j - m_i) for j <= i
//   mode  U        W        (i,j)   X        A        rowscale        Bm
//   H     Q        K        (r,c)   V        Q        qk_scale*bbar   C_k[a][o]
//   DV    K        Q        (c,r)   dHbar    K        abar            dC_{k+1}[a][o]
//   DK    V        dHbar    (c,r)   Q        V        abar            dC_{k+1}[o][a]
//   DQ    dHbar    V        (r,c)   K        dHbar    qk_scale*bbar   C_k[o][a]
// dHbar = deltaH / (den + eps).  grid (ceil(DO/64), ceil(L/64), B*NH*NC)
// =====================================================================================================
enum { PAR_H = 0, PAR_DV = 1, PAR_DK = 2, PAR_DQ = 3 };

template <typename T, typename TS>
struct ParArgs {
  const T *q, *k, *v, *dh;
  const float *vecB, *iota, *m_tok, *abar, *bbar, *inv_den;
  const TS* c_states;   // slot k used by H and DQ
  const TS* dc_states;  // slot k+1 used by DV and DK
  const float* n_states;
  void* out;     // T*
  float* n_out;  // H only
  int S, L, NC, DHQK, DHHV, variant;
  float eps, qk_scale;
};

template <typename T, typename TS, int MODE>
__global__ void __launch_bounds__(NTHR) par_kernel(ParArgs<T, TS> p) {
  extern __shared__ float smem[];
  const int L = p.L;
  float* s_b = smem;              // [L]
  float* s_iota = s_b + L;        // [L]
  float* s_m = s_iota + L;        // [L]
  float* Us = s_m + L;            // [64][33]   (also As)
  float* Ws = Us + TILE * (KSL + 1);  // [64][33]
  float* Ps = Ws + TILE * (KSL + 1);  // [64][65]
  float* Xs = Ps + TILE * (TILE + 1);  // [64][65]  (also Bs [32][65])
  float* s_row = Xs + TILE * (TILE + 1);  // [64] row sums / denominators
  float* s_qn = s_row + TILE;             // [64]
  float* s_n = s_qn + TILE;               // [32]

  const int tid = threadIdx.x, tx = tid & 15, ty = tid >> 4;
  // grid (output tiles x chunks x batch x heads, row blocks): the large factor sits in x, which has no 65535 limit
  const int n_ot = (((MODE == PAR_H || MODE == PAR_DV) ? p.DHHV : p.DHQK) + TILE - 1) / TILE;
  const int ot = blockIdx.x % n_ot, bc = blockIdx.x / n_ot;
  const int o0 = ot * TILE, rb = blockIdx.y, r0 = rb * TILE;
  const int bh = bc / p.NC, ck = bc % p.NC;
  const size_t tok0 = (size_t)bh * p.S + (size_t)ck * L;
  constexpr bool LOWER = (MODE == PAR_H || MODE == PAR_DQ);
  const int DI = (MODE == PAR_H || MODE == PAR_DV) ? p.DHQK : p.DHHV;   // contraction dim of P
  const int DO = (MODE == PAR_H || MODE == PAR_DV) ? p.DHHV : p.DHQK;   // output width
  const int DA = (MODE == PAR_H || MODE == PAR_DV) ? p.DHQK : p.DHHV;   // contraction dim of the inter term

  // element accessors (value of matrix `which` at chunk row r, column c; zero outside)
  auto ldU = [&](int r, int c) -> float {
    if (r >= L || c >= DI) return 0.f;
    const size_t t = tok0 + r;
    if (MODE == PAR_H) return to_f32(p.q[t * p.DHQK + c]);
    if (MODE == PAR_DV) return to_f32(p.k[t * p.DHQK + c]);
    if (MODE == PAR_DK) return to_f32(p.v[t * p.DHHV + c]);
    return to_f32(p.dh[t * p.DHHV + c]) * p.inv_den[t];
  };
  auto ldW = [&](int r, int c) -> float {
    if (r >= L || c >= DI) return 0.f;
    const size_t t = tok0 + r;
    if (MODE == PAR_H) return to_f32(p.k[t * p.DHQK + c]);
    if (MODE == PAR_DV) return to_f32(p.q[t * p.DHQK + c]);
    if (MODE == PAR_DK) return to_f32(p.dh[t * p.DHHV + c]) * p.inv_den[t];
    return to_f32(p.v[t * p.DHHV + c]);
  };
  auto ldX = [&](int r, int c) -> float {
    if (r >= L || c >= DO) return 0.f;
    const size_t t = tok0 + r;
    if (MODE == PAR_H) return to_f32(p.v[t * p.DHHV + c]);
    if (MODE == PAR_DV) return to_f32(p.dh[t * p.DHHV + c]) * p.inv_den[t];
    if (MODE == PAR_DK) return to_f32(p.q[t * p.DHQK + c]);
    return to_f32(p.k[t * p.DHQK + c]);
  };

  for (int j = tid; j < L; j += NTHR) {
    s_b[j] = p.vecB[tok0 + j];
    s_iota[j] = p.iota[tok0 + j];
    s_m[j] = p.m_tok[tok0 + j];
  }
  if (tid < TILE) { s_row[tid] = 0.f; s_qn[tid] = 0.f; }
  __syncthreads();

  float acc[4][4] = {};
  float rowsum = 0.f;
  const int nblk = (L + TILE - 1) / TILE;
  const int cb_lo = LOWER ? 0 : rb, cb_hi = LOWER ? rb : nblk - 1;
  for (int cb = cb_lo; cb <= cb_hi; ++cb) {
    const int c0 = cb * TILE;
    float pr[4][4] = {};
    for (int di0 = 0; di0 < DI; di0 += KSL) {
      for (int idx = tid; idx < TILE * KSL; idx += NTHR) {
        const int r = idx / KSL, c = idx % KSL;
        Us[r * (KSL + 1) + c] = ldU(r0 + r, di0 + c);
        Ws[r * (KSL + 1) + c] = ldW(c0 + r, di0 + c);
      }
      __syncthreads();
#pragma unroll 8
      for (int d = 0; d < KSL; ++d) {
        float a4[4], b4[4];
#pragma unroll
        for (int a = 0; a < 4; ++a) a4[a] = Us[(ty * 4 + a) * (KSL + 1) + d];
#pragma unroll
        for (int b = 0; b < 4; ++b) b4[b] = Ws[(tx * 4 + b) * (KSL + 1) + d];
#pragma unroll
        for (int a = 0; a < 4; ++a)
#pragma unroll
          for (int b = 0; b < 4; ++b) pr[a][b] = fmaf(a4[a], b4[b], pr[a][b]);
      }
      __syncthreads();
    }
#pragma unroll
    for (int a = 0; a < 4; ++a)
#pragma unroll
      for (int b = 0; b < 4; ++b) {
        const int r = r0 + ty * 4 + a, c = c0 + tx * 4 + b;
        const bool valid = (r < L) && (c < L) && (LOWER ? (c <= r) : (c >= r));
        float val = 0.f;
        if (valid) {
          const int ii = LOWER ? r : c, jj = LOWER ? c : r;
          val = p.qk_scale * pr[a][b] * expf((s_b[ii] - s_b[jj]) + s_iota[jj] - s_m[ii]);
        }
        Ps[(ty * 4 + a) * (TILE + 1) + tx * 4 + b] = val;
      }
    for (int idx = tid; idx < TILE * TILE; idx += NTHR) {
      const int r = idx / TILE, c = idx % TILE;
      Xs[r * (TILE + 1) + c] = ldX(c0 + r, o0 + c);
    }
    __syncthreads();
#pragma unroll 8
    for (int c = 0; c < TILE; ++c) {
      float a4[4], b4[4];
#pragma unroll
      for (int a = 0; a < 4; ++a) a4[a] = Ps[(ty * 4 + a) * (TILE + 1) + c];
#pragma unroll
      for (int b = 0; b < 4; ++b) b4[b] = Xs[c * (TILE + 1) + tx * 4 + b];
#pragma unroll
      for (int a = 0; a < 4; ++a)
#pragma unroll
        for (int b = 0; b < 4; ++b) acc[a][b] = fmaf(a4[a], b4[b], acc[a][b]);
    }
    if (MODE == PAR_H && tid < TILE) {
      for (int c = 0; c < TILE; ++c) rowsum += Ps[tid * (TILE + 1) + c];
    }
    __syncthreads();
  }

  // ---- inter-chunk contribution ----
  float acc2[4][4] = {};
  float qn = 0.f;
  const TS* Bsrc = (MODE == PAR_H || MODE == PAR_DQ)
                       ? p.c_states + ((size_t)bh * (p.NC + 1) + ck) * p.DHQK * p.DHHV
                       : p.dc_states + ((size_t)bh * (p.NC + 1) + ck + 1) * p.DHQK * p.DHHV;
  const float* nsrc = (MODE == PAR_H && p.n_states) ? p.n_states + ((size_t)bh * (p.NC + 1) + ck) * p.DHQK : nullptr;
  float* As = Us;
  float* Bs = Xs;
  for (int da0 = 0; da0 < DA; da0 += KSL) {
    for (int idx = tid; idx < TILE * KSL; idx += NTHR) {
      const int r = idx / KSL, c = idx % KSL;
      As[r * (KSL + 1) + c] = ldU(r0 + r, da0 + c);  // A is the same matrix as U in every mode
    }
    if (MODE == PAR_H || MODE == PAR_DV) {
      for (int idx = tid; idx < KSL * TILE; idx += NTHR) {
        const int a = idx / TILE, o = idx % TILE;
        float val = 0.f;
        if (da0 + a < DA && o0 + o < DO) val = to_f32(Bsrc[(size_t)(da0 + a) * p.DHHV + o0 + o]);
        Bs[a * (TILE + 1) + o] = val;
      }
    } else {
      for (int idx = tid; idx < KSL * TILE; idx += NTHR) {
        const int a = idx % KSL, o = idx / KSL;
        float val = 0.f;
        if (da0 + a < DA && o0 + o < DO) val = to_f32(Bsrc[(size_t)(o0 + o) * p.DHHV + da0 + a]);
        Bs[a * (TILE + 1) + o] = val;
      }
    }
    if (MODE == PAR_H && tid < KSL) s_n[tid] = (nsrc && da0 + tid < DA) ? nsrc[da0 + tid] : 0.f;
    __syncthreads();
#pragma unroll 8
    for (int d = 0; d < KSL; ++d) {
      float a4[4], b4[4];
#pragma unroll
      for (int a = 0; a < 4; ++a) a4[a] = As[(ty * 4 + a) * (KSL + 1) + d];
#pragma unroll
      for (int b = 0; b < 4; ++b) b4[b] = Bs[d * (TILE + 1) + tx * 4 + b];
#pragma unroll
      for (int a = 0; a < 4; ++a)
#pragma unroll
        for (int b = 0; b < 4; ++b) acc2[a][b] = fmaf(a4[a], b4[b], acc2[a][b]);
    }
    if (MODE == PAR_H && tid < TILE) {
      for (int d = 0; d < KSL; ++d) qn = fmaf(As[tid * (KSL + 1) + d], s_n[d], qn);
    }
    __syncthreads();
  }

  // ---- epilogue ----
  if (MODE == PAR_H && tid < TILE) {
    const int r = r0 + tid;
    float den = 1.f;
    if (r < L) {
      const float nn = rowsum + p.qk_scale * p.bbar[tok0 + r] * qn;
      if (p.variant == MLSTM_EXP) den = fmaxf(fabsf(nn), expf(-s_m[r]));
      else if (p.variant == MLSTM_SIG) den = fmaxf(fabsf(nn), 1.f);
      if (ot == 0) p.n_out[tok0 + r] = den;
    }
    s_row[tid] = den;
  }
  __syncthreads();
  T* out = (T*)p.out;
#pragma unroll
  for (int a = 0; a < 4; ++a) {
    const int r = r0 + ty * 4 + a;
    if (r >= L) continue;
    const size_t t = tok0 + r;
    float rs;
    if (MODE == PAR_H || MODE == PAR_DQ) rs = p.qk_scale * p.bbar[t];
    else rs = p.abar[t];
#pragma unroll
    for (int b = 0; b < 4; ++b) {
      const int o = o0 + tx * 4 + b;
      if (o >= DO) continue;
      float val = acc[a][b] + rs * acc2[a][b];
      if (MODE == PAR_H && p.variant != MLSTM_SIG_NONORM) val = val / (s_row[ty * 4 + a] + p.eps);
      out[t * DO + o] = from_f32<T>(val);
    }
  }
}

static size_t par_smem_bytes(int L) {
  return sizeof(float) * ((size_t)3 * L + 2 * TILE * (KSL + 1) + 2 * TILE * (TILE + 1) + 2 * TILE + KSL);
}

// ---- launchers ----------------------------------------------------------------------------------------
template <typename T, typename TS>
int rec_fw_t(const void* k, const void* v, const GateBuffers& gb, const float* c_initial, const float* n_initial,
             void* c_states, float* n_states, float* c_last, float* n_last, const ChunkwiseDims& d, cudaStream_t st) {
  PhaseScope ps(PH_REC_FW, st);
  dim3 grid(ceil_div(d.DHHV, TILE) * d.B * d.NH, ceil_div(d.DHQK, TILE));
  rec_kernel<T, TS, false><<<grid, NTHR, 0, st>>>((const T*)k, (const T*)v, gb.abar, 1.f, nullptr, gb.gbar, c_initial,
                                                  n_initial, (TS*)c_states, n_states, c_last, n_last, d.S, d.L, d.NC,
                                                  d.DHQK, d.DHHV);
  MLSTM_LAUNCH_CHECK();
  return MLSTM_OK;
}
template <typename T, typename TS>
int rec_bw_t(const void* q, const void* dh, const GateBuffers& gb, const float* dc_last, void* dc_states,
             float* dc_initial, const ChunkwiseDims& d, cudaStream_t st) {
  PhaseScope ps(PH_REC_BW, st);
  dim3 grid(ceil_div(d.DHHV, TILE) * d.B * d.NH, ceil_div(d.DHQK, TILE));
  rec_kernel<T, TS, true><<<grid, NTHR, 0, st>>>((const T*)q, (const T*)dh, gb.bbar, d.qk_scale, gb.inv_den, gb.gbar,
                                                 dc_last, nullptr, (TS*)dc_states, nullptr, dc_initial, nullptr, d.S,
                                                 d.L, d.NC, d.DHQK, d.DHHV);
  MLSTM_LAUNCH_CHECK();
  return MLSTM_OK;
}

template <typename T, typename TS, int MODE>
int par_launch(ParArgs<T, TS>& a, const ChunkwiseDims& d, cudaStream_t st) {
  const int DO = (MODE == PAR_H || MODE == PAR_DV) ? d.DHHV : d.DHQK;
  const size_t smem = par_smem_bytes(d.L);
  auto kern = par_kernel<T, TS, MODE>;
  MLSTM_CUDA_CHECK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
  dim3 grid(ceil_div(DO, TILE) * d.B * d.NH * d.NC, ceil_div(d.L, TILE));
  kern<<<grid, NTHR, smem, st>>>(a);
  MLSTM_LAUNCH_CHECK();
  return MLSTM_OK;
}

template <typename T, typename TS>
ParArgs<T, TS> make_args(const void* q, const void* k, const void* v, const void* dh, const GateBuffers& gb,
                         const void* c_states, const void* dc_states, const float* n_states, const ChunkwiseDims& d) {
  ParArgs<T, TS> a;
  a.q = (const T*)q; a.k = (const T*)k; a.v = (const T*)v; a.dh = (const T*)dh;
  a.vecB = gb.vecB; a.iota = gb.iota; a.m_tok = gb.m_tok; a.abar = gb.abar; a.bbar = gb.bbar; a.inv_den = gb.inv_den;
  a.c_states = (const TS*)c_states; a.dc_states = (const TS*)dc_states; a.n_states = n_states;
  a.out = nullptr; a.n_out = nullptr;
  a.S = d.S; a.L = d.L; a.NC = d.NC; a.DHQK = d.DHQK; a.DHHV = d.DHHV; a.variant = d.variant;
  a.eps = d.eps; a.qk_scale = d.qk_scale;
  return a;
}

template <typename T, typename TS>
int par_fw_t(const void* q, const void* k, const void* v, const GateBuffers& gb, const void* c_states,
             const float* n_states, void* h, float* n_out, const ChunkwiseDims& d, cudaStream_t st) {
  auto a = make_args<T, TS>(q, k, v, nullptr, gb, c_states, nullptr, n_states, d);
  a.out = h; a.n_out = n_out;
  PhaseScope ps(PH_PAR_FW, st);
  return par_launch<T, TS, PAR_H>(a, d, st);
}
template <typename T, typename TS>
int par_bw_t(const void* q, const void* k, const void* v, const void* dh, const GateBuffers& gb, const void* c_states,
             const void* dc_states, void* dq, void* dk, void* dv, const ChunkwiseDims& d, cudaStream_t st) {
  auto a = make_args<T, TS>(q, k, v, dh, gb, c_states, dc_states, nullptr, d);
  int rc;
  PhaseScope ps(PH_PAR_BW, st);
  a.out = dv; if ((rc = par_launch<T, TS, PAR_DV>(a, d, st)) != MLSTM_OK) return rc;
  a.out = dk; if ((rc = par_launch<T, TS, PAR_DK>(a, d, st)) != MLSTM_OK) return rc;
  a.out = dq; if ((rc = par_launch<T, TS, PAR_DQ>(a, d, st)) != MLSTM_OK) return rc;
  return MLSTM_OK;
}

#define MLSTM_DISPATCH(dtype, state_dtype, FN, ...)                                                      \
  do {                                                                                                   \
    if (state_dtype == MLSTM_F32) {                                                                      \
      if (dtype == MLSTM_F32) return FN<float, float>(__VA_ARGS__);                                      \
      if (dtype == MLSTM_BF16) return FN<__nv_bfloat16, float>(__VA_ARGS__);                             \
      if (dtype == MLSTM_F16) return FN<__half, float>(__VA_ARGS__);                                     \
    } else if (state_dtype == MLSTM_BF16) {                                                              \
      if (dtype == MLSTM_BF16) return FN<__nv_bfloat16, __nv_bfloat16>(__VA_ARGS__);                     \
    }                                                                                                    \
    return MLSTM_ERR_DTYPE;                                                                              \
  } while (0)

int simt_recurrent_fw(int dtype, int state_dtype, const void* k, const void* v, const GateBuffers& gb,
                      const float* c_initial, const float* n_initial, void* c_states, float* n_states,
                      float* c_last, float* n_last, const ChunkwiseDims& d, cudaStream_t st) {
  MLSTM_DISPATCH(dtype, state_dtype, rec_fw_t, k, v, gb, c_initial, n_initial, c_states, n_states, c_last, n_last, d, st);
}
int simt_parallel_fw(int dtype, int state_dtype, const void* q, const void* k, const void* v, const GateBuffers& gb,
                     const void* c_states, const float* n_states, void* h, float* n_out, const ChunkwiseDims& d,
                     cudaStream_t st) {
  MLSTM_DISPATCH(dtype, state_dtype, par_fw_t, q, k, v, gb, c_states, n_states, h, n_out, d, st);
}
int simt_recurrent_bw(int dtype, int state_dtype, const void* q, const void* dh, const GateBuffers& gb,
                      const float* dc_last, void* dc_states, float* dc_initial, const ChunkwiseDims& d,
                      cudaStream_t st) {
  MLSTM_DISPATCH(dtype, state_dtype, rec_bw_t, q, dh, gb, dc_last, dc_states, dc_initial, d, st);
}
int simt_parallel_bw(int dtype, int state_dtype, const void* q, const void* k, const void* v, const void* dh,
                     const GateBuffers& gb, const void* c_states, const void* dc_states, void* dq, void* dk, void* dv,
                     const ChunkwiseDims& d, cudaStream_t st) {
  MLSTM_DISPATCH(dtype, state_dtype, par_bw_t, q, k, v, dh, gb, c_states, dc_states, dq, dk, dv, d, st);
}

}  // namespace mlstm
