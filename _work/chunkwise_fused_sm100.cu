// Fused chunkwise forward for B200: the inter-chunk state stays on chip.
//
// One persistent CTA per (batch, head, 128-column slice of DHHV) walks the chunks of the sequence in order and does
// the inter-chunk recurrence and the intra-chunk output together, so the f32 state C never makes a round trip
// through HBM between the two (the bf16 per-chunk states are still written out, once, for the backward pass):
//   tensor memory (512 columns): C[0:128,:] | C[128:256,:] | score tile S | output accumulator
//   shared memory: bf16 copy of C (B operand of Q.C), the K chunk, the V tile, a two-stage ring of Q slices
// Per chunk k (L = 128 tokens, DHQK = 256):
//   S   = Q K^T                      16 MMAs   (ring slice d: Q_d with K box d)
//   Acc = Q Cbf_{k-1}                16 MMAs   (same Q slice, B = bf16 state in shared memory)
//   K  <- abar (.) K in place        CUDA cores (after S has read K); n_k from the column sums
//   C   = gbar_k C + Kbar^T V        16 MMAs accumulating onto the pre-scaled state in tensor memory
//   S  -> gate, causal mask -> bf16  CUDA cores, tensor memory to tensor memory; Acc row-scaled in place
//   Acc += Sbar V                     8 MMAs;  H = Acc / den
//   state pass: C_k -> bf16 copy in shared memory (+ TMA store to the state buffer), C <- gbar_{k+1} C
// Math: mlstm_kernels/triton/chunkwise/xl_chunk/fw_kernel_recurrent.py:14-230 and fw_kernel_parallel.py:14-289.
// Warps: 0 TMA producer, 1 MMA issuer, 2..9 gate/epilogue (thread = output row), 10..13 K scaling and n,
// 14..21 state pass.  Every wait is bounded (status word g_sm100_status, codes 3xx).
#include "common.cuh"
#include "launch.cuh"
#include "sm100.cuh"

namespace mlstm {

using namespace sm100;

extern __device__ int g_sm100_status;

constexpr int FL = 128;            // chunk length
constexpr int FDQK = 256;          // DHQK handled by this kernel
constexpr int F_THREADS = 704;
constexpr int F_NQ = 2;            // Q ring stages
constexpr int F_OFF_C = 0;                       // bf16 state copy: 4 slices x 2 boxes x 8 KB
constexpr int F_OFF_K = 65536;                   // K chunk: 4 boxes of 128 rows x 64 columns
constexpr int F_OFF_V = 131072;                  // V tile: 2 boxes of 128 rows x 64 columns
constexpr int F_OFF_Q = 163840;                  // Q ring: F_NQ slices of 16 KB
constexpr int F_OFF_NP = F_OFF_Q + F_NQ * 16384;  // partial column sums for n: 16 row groups x 256 columns, f32
constexpr int F_SMEM = F_OFF_NP + 16 * 256 * 4 + 1024;

struct FusedParams {
  const float *vecB, *iota, *m_tok, *abar, *bbar, *gbar;   // gate pre-pass output
  const float *c_init, *n_init;                              // (BNH, DHQK, DHHV), (BNH, DHQK) or nullptr
  __nv_bfloat16* h;                                          // (BNH*S, DHHV)
  float* n_out;                                              // (BNH*S)
  float* n_states;                                           // (BNH, NC+1, DHQK) or nullptr
  float *c_last, *n_last;                                    // f32 final state or nullptr
  int store_states;                                          // write the bf16 per-chunk states through mapCs
  int S, NC, DHHV, variant;
  float eps, qk_scale;
};

struct FusedShared {
  uint64_t kfull, kfree, vfull, vfree, qfull[F_NQ], qempty[F_NQ];
  uint64_t sfull, gated, hfull, accfree, kscaled, pfull, cready, cstore, nsum, nready, colready, pair[4];
  uint32_t tmem;
  float s_scale[2][FL];      // abar of the chunk's rows (staged by the producer warp)
  float s_colA[2][FL];       // iota_j - b_j of the chunk's columns
  float s_n[2][FDQK];        // n_{k-1} for chunk k
  float s_part[2][FL], s_qn[2][FL];
};

__global__ void __launch_bounds__(F_THREADS, 1)
fused_fw_sm100(const __grid_constant__ CUtensorMap mapQ, const __grid_constant__ CUtensorMap mapK,
               const __grid_constant__ CUtensorMap mapV, const __grid_constant__ CUtensorMap mapCs,
               const __grid_constant__ FusedParams p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  __shared__ FusedShared sh;

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int e0 = blockIdx.x * 128, bh = blockIdx.y;
  const int NC = p.NC;
  const bool use_n = p.variant != MLSTM_SIG_NONORM;
  int* const err = &g_sm100_status;

  if (tid == 0) {
    mbar_init(&sh.kfull, 1); mbar_init(&sh.kfree, 1); mbar_init(&sh.vfull, 1); mbar_init(&sh.vfree, 1);
    for (int s = 0; s < F_NQ; ++s) { mbar_init(&sh.qfull[s], 1); mbar_init(&sh.qempty[s], use_n ? 9 : 1); }
    mbar_init(&sh.sfull, 1); mbar_init(&sh.gated, 256); mbar_init(&sh.hfull, 1); mbar_init(&sh.accfree, 256);
    mbar_init(&sh.kscaled, 128); mbar_init(&sh.pfull, 1); mbar_init(&sh.cready, 256); mbar_init(&sh.cstore, 1);
    mbar_init(&sh.nsum, 128); mbar_init(&sh.nready, 128); mbar_init(&sh.colready, 256);
    for (int s = 0; s < 4; ++s) mbar_init(&sh.pair[s], 64);
    fence_barrier_init();
    tma_prefetch_desc(&mapQ); tma_prefetch_desc(&mapK); tma_prefetch_desc(&mapV); tma_prefetch_desc(&mapCs);
  }
  if (warp == 1) { tmem_alloc(&sh.tmem, 512); tmem_relinquish(); }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem = sh.tmem;
  const uint32_t tC0 = tmem, tC1 = tmem + 128, tS = tmem + 256, tAcc = tmem + 384;

  if (warp == 0) {
    // =============================== TMA producer ===============================
    bool ok = true;
    float ab_next[4];
#pragma unroll
    for (int u = 0; u < 4; ++u) ab_next[u] = (NC > 0) ? p.abar[(size_t)bh * p.S + lane + 32 * u] : 0.f;
    for (int k = 0; k < NC && ok; ++k) {
      const int row0 = bh * p.S + k * FL;
      float ab[4];
#pragma unroll
      for (int u = 0; u < 4; ++u) ab[u] = ab_next[u];
      if (k + 1 < NC) {   // fetched before the wait below, so the latency is not on the load path
#pragma unroll
        for (int u = 0; u < 4; ++u) ab_next[u] = p.abar[(size_t)row0 + FL + lane + 32 * u];
      }
      // K chunk: needs the previous chunk's state-update MMAs (the last readers of the K buffer) to be done
      int okw = 1;
      if (lane == 0 && k > 0) okw = mbar_wait(&sh.kfree, (k - 1) & 1, err, 301) ? 1 : 0;
      okw = __shfl_sync(0xffffffffu, okw, 0);
      if (!okw) { ok = false; break; }
      // per-row scales of this chunk; their buffer (parity k) was last read while chunk k-2 was being scaled
#pragma unroll
      for (int u = 0; u < 4; ++u) sh.s_scale[k & 1][lane + 32 * u] = ab[u];
      __syncwarp();
      if (lane == 0) {
        mbar_expect_tx(&sh.kfull, 65536);
#pragma unroll
        for (int b = 0; b < 4; ++b) tma_load_2d(smem + F_OFF_K + b * 16384, &mapK, &sh.kfull, 64 * b, row0);
        for (int d4 = 0; d4 < 4 && ok; ++d4) {
          const int j = k * 4 + d4, st = j % F_NQ;
          if (!mbar_wait(&sh.qempty[st], ((j / F_NQ) & 1) ^ 1, err, 302)) { ok = false; break; }
          mbar_expect_tx(&sh.qfull[st], 16384);
          tma_load_2d(smem + F_OFF_Q + st * 16384, &mapQ, &sh.qfull[st], 64 * d4, row0);
        }
        if (ok && k > 0) ok = mbar_wait(&sh.vfree, (k - 1) & 1, err, 303);
        if (ok) {
          mbar_expect_tx(&sh.vfull, 32768);
          tma_load_2d(smem + F_OFF_V, &mapV, &sh.vfull, e0, row0);
          tma_load_2d(smem + F_OFF_V + 16384, &mapV, &sh.vfull, e0 + 64, row0);
        }
      }
      ok = __shfl_sync(0xffffffffu, ok ? 1 : 0, 0) != 0;
    }
    // error path: copies that were issued land within a bounded time; wait for the last ones before retiring
    if (!ok && lane == 0) {
      int dummy = 1;
      for (uint32_t it = 0; it < 200000u; ++it) { __nanosleep(64); (void)dummy; }
    }
  } else if (warp == 1) {
    // =============================== MMA issuer ===============================
    if (lane == 0) {
      constexpr uint32_t id_kk = umma_idesc_bf16(128, 128, 0, 0);   // A K-major, B K-major
      constexpr uint32_t id_kn = umma_idesc_bf16(128, 128, 0, 1);   // A K-major (or tensor memory), B MN-major
      constexpr uint32_t id_nn = umma_idesc_bf16(128, 128, 1, 1);   // both MN-major
      const uint32_t sC = smem_u32(smem + F_OFF_C), sK = smem_u32(smem + F_OFF_K), sV = smem_u32(smem + F_OFF_V);
      bool ok = true;
      for (int k = 0; k < NC && ok; ++k) {
        // Q.K^T and Q.C_{k-1}: need K_k, the state pass of chunk k-1 (index k in the cready sequence, the
        // initial state being pass 0) and the output accumulator released by the epilogue of chunk k-1
        ok = mbar_wait(&sh.kfull, k & 1, err, 311) && mbar_wait(&sh.cready, k & 1, err, 312);
        if (ok && k > 0) ok = mbar_wait(&sh.accfree, (k - 1) & 1, err, 313);
        if (!ok) break;
        for (int d4 = 0; d4 < 4; ++d4) {
          const int j = k * 4 + d4, st = j % F_NQ;
          if (!mbar_wait(&sh.qfull[st], (j / F_NQ) & 1, err, 314)) { ok = false; break; }
          tc_fence_after_sync();
          const uint32_t sq = smem_u32(smem + F_OFF_Q + st * 16384);
#pragma unroll
          for (int kk = 0; kk < 4; ++kk)
            umma_ss(tS, umma_desc_sw128(sq + kk * 32, 16, 1024), umma_desc_sw128(sK + d4 * 16384 + kk * 32, 16, 1024),
                    id_kk, (d4 > 0 || kk > 0) ? 1u : 0u);
#pragma unroll
          for (int kk = 0; kk < 4; ++kk)
            umma_ss(tAcc, umma_desc_sw128(sq + kk * 32, 16, 1024),
                    umma_desc_sw128(sC + d4 * 16384 + kk * 2048, 8192, 1024), id_kn, (d4 > 0 || kk > 0) ? 1u : 0u);
          umma_commit(&sh.qempty[st]);
        }
        if (!ok) break;
        umma_commit(&sh.sfull);
        // state update C += Kbar^T V (the state in tensor memory already carries the decay of this chunk)
        ok = mbar_wait(&sh.kscaled, k & 1, err, 315) && mbar_wait(&sh.vfull, k & 1, err, 316);
        if (!ok) break;
        tc_fence_after_sync();
#pragma unroll
        for (int mh = 0; mh < 2; ++mh)
#pragma unroll
          for (int kk = 0; kk < 8; ++kk)
            umma_ss(mh ? tC1 : tC0, umma_desc_sw128(sK + mh * 32768 + kk * 2048, 16384, 1024),
                    umma_desc_sw128(sV + kk * 2048, 16384, 1024), id_nn, 1u);
        umma_commit(&sh.pfull);
        umma_commit(&sh.kfree);
        // intra-chunk product on the gated scores
        if (!mbar_wait(&sh.gated, k & 1, err, 317)) { ok = false; break; }
        tc_fence_after_sync();
#pragma unroll
        for (int kk = 0; kk < 8; ++kk)
          umma_ts(tAcc, tS + kk * 8, umma_desc_sw128(sV + kk * 2048, 16384, 1024), id_kn, 1u);
        umma_commit(&sh.hfull);
        umma_commit(&sh.vfree);
      }
    }
  } else if (warp < 10) {
    // =============================== gate / epilogue warps ===============================
    const int quarter = warp & 3, half = (warp - 2) >> 2;
    const int r = quarter * 32 + lane;
    const uint32_t lane_base = (uint32_t)(quarter * 32) << 16;
    bool ok = true;
    // per-row gate values are fetched one chunk ahead
    float nb_r = 0.f, ni_r = 0.f, nm_r = 0.f, nbb_r = 0.f;
    if (NC > 0) {
      const size_t t0 = (size_t)bh * p.S + r;
      nb_r = p.vecB[t0]; ni_r = p.iota[t0]; nm_r = p.m_tok[t0]; nbb_r = p.bbar[t0];
    }
    for (int k = 0; k < NC && ok; ++k) {
      const size_t tok = (size_t)bh * p.S + (size_t)k * FL + r;
      const float b_r = nb_r, iota_r = ni_r, m_r = nm_r, bbar_r = nbb_r;
      if (k + 1 < NC) { nb_r = p.vecB[tok + FL]; ni_r = p.iota[tok + FL]; nm_r = p.m_tok[tok + FL]; nbb_r = p.bbar[tok + FL]; }
      const float rowA = b_r - m_r;
      const float rowscale = p.qk_scale * bbar_r;
      float* colA = sh.s_colA[k & 1];
      if (half == 0) colA[r] = iota_r - b_r;
      mbar_arrive(&sh.colready);
      // q . n_{k-1}: read this thread's half row of every Q slice from the ring
      float qn = 0.f;
      if (use_n) {
        if (!mbar_wait(&sh.nready, k & 1, err, 321)) { ok = false; break; }   // phase k: n before chunk k is in s_n[k & 1]
        const float* nsm = sh.s_n[k & 1];
        for (int d4 = 0; d4 < 4; ++d4) {
          const int j = k * 4 + d4, st = j % F_NQ;
          if (!mbar_wait(&sh.qfull[st], (j / F_NQ) & 1, err, 322)) { ok = false; break; }
          const uint8_t* rowp = smem + F_OFF_Q + st * 16384 + r * 128;
#pragma unroll
          for (int cc = 0; cc < 4; ++cc) {
            const int lc = half * 4 + cc;
            const uint4 v = *reinterpret_cast<const uint4*>(rowp + ((lc ^ (r & 7)) << 4));
            const uint32_t w[4] = {v.x, v.y, v.z, v.w};
            const float* nn = nsm + d4 * 64 + lc * 8;
#pragma unroll
            for (int e = 0; e < 4; ++e) {
              const __nv_bfloat162 h2 = *reinterpret_cast<const __nv_bfloat162*>(&w[e]);
              qn = fmaf(__low2float(h2), nn[2 * e], qn);
              qn = fmaf(__high2float(h2), nn[2 * e + 1], qn);
            }
          }
          __syncwarp();
          if (lane == 0) mbar_arrive(&sh.qempty[st]);
        }
        if (!ok) break;
        sh.s_qn[half][r] = qn;
      }
      ok = mbar_wait(&sh.colready, k & 1, err, 323) && mbar_wait(&sh.sfull, k & 1, err, 324);
      if (!ok) break;
      tc_fence_after_sync();
      // row-scale the inter-chunk term in place
#pragma unroll 1
      for (int cq = half; cq < 4; cq += 2) {
        uint32_t v[32];
        tmem_ld32(tAcc + lane_base + cq * 32, v);
        tmem_wait_ld();
#pragma unroll
        for (int c = 0; c < 32; ++c) v[c] = __float_as_uint(__uint_as_float(v[c]) * rowscale);
        tmem_st32(tAcc + lane_base + cq * 32, v);
      }
      // gate the scores (lower triangle), bf16 back to tensor memory
      float rowsum = 0.f;
      uint32_t pk[2][16];
#pragma unroll
      for (int u = 0; u < 2; ++u) {
        const int cq = half + 2 * u, c0 = cq * 32;
        if (cq > quarter) {
#pragma unroll
          for (int c = 0; c < 16; ++c) pk[u][c] = 0u;
        } else {
          uint32_t v[32];
          tmem_ld32(tS + lane_base + c0, v);
          tmem_wait_ld();
          const bool diag = (cq == quarter);
#pragma unroll
          for (int c = 0; c < 16; ++c) {
            float g2[2];
#pragma unroll
            for (int h = 0; h < 2; ++h) {
              const int cl = 2 * c + h;
              float val = __uint_as_float(v[cl]) * p.qk_scale * __expf(rowA + colA[c0 + cl]);
              if (diag && cl > lane) val = 0.f;
              g2[h] = val;
              rowsum += val;
            }
            pk[u][c] = pack_bf16(g2[0], g2[1]);
          }
        }
      }
      tc_fence_before_sync();
      mbar_arrive(&sh.pair[quarter]);
      if (!mbar_wait(&sh.pair[quarter], k & 1, err, 325)) { ok = false; break; }
      tc_fence_after_sync();
#pragma unroll
      for (int u = 0; u < 2; ++u) tmem_st16(tS + lane_base + (half + 2 * u) * 16, pk[u]);
      sh.s_part[half][r] = rowsum;
      tmem_wait_st();
      tc_fence_before_sync();
      mbar_arrive(&sh.gated);
      if (!mbar_wait(&sh.hfull, k & 1, err, 326)) { ok = false; break; }
      tc_fence_after_sync();
      float inv = 1.f, den = 1.f;
      const float nn = (sh.s_part[0][r] + sh.s_part[1][r]) + rowscale * (use_n ? (sh.s_qn[0][r] + sh.s_qn[1][r]) : 0.f);
      if (p.variant == MLSTM_EXP) den = fmaxf(fabsf(nn), __expf(-m_r));
      else if (p.variant == MLSTM_SIG) den = fmaxf(fabsf(nn), 1.f);
      if (p.variant != MLSTM_SIG_NONORM) inv = 1.f / (den + p.eps);
      if (blockIdx.x == 0 && half == 0) p.n_out[tok] = den;
      __nv_bfloat16* orow = p.h + tok * p.DHHV + e0;
#pragma unroll 1
      for (int cq = half; cq < 4; cq += 2) {
        uint32_t v[32];
        tmem_ld32(tAcc + lane_base + cq * 32, v);
        tmem_wait_ld();
        uint4* dst = reinterpret_cast<uint4*>(orow + cq * 32);
#pragma unroll
        for (int c = 0; c < 4; ++c) {
          uint4 o;
          o.x = pack_bf16(__uint_as_float(v[8 * c]) * inv, __uint_as_float(v[8 * c + 1]) * inv);
          o.y = pack_bf16(__uint_as_float(v[8 * c + 2]) * inv, __uint_as_float(v[8 * c + 3]) * inv);
          o.z = pack_bf16(__uint_as_float(v[8 * c + 4]) * inv, __uint_as_float(v[8 * c + 5]) * inv);
          o.w = pack_bf16(__uint_as_float(v[8 * c + 6]) * inv, __uint_as_float(v[8 * c + 7]) * inv);
          dst[c] = o;
        }
      }
      tc_fence_before_sync();
      mbar_arrive(&sh.accfree);
    }
  } else if (warp < 14) {
    // =============================== K scaling warps (and n) ===============================
    const int t = tid - 320;   // 0..127
    float n0v = 0.f, n1v = 0.f;   // n columns 2t, 2t+1
    const bool n_owner = use_n && blockIdx.x == 0;
    if (use_n && p.n_init) { n0v = p.n_init[(size_t)bh * FDQK + 2 * t]; n1v = p.n_init[(size_t)bh * FDQK + 2 * t + 1]; }
    if (use_n) { sh.s_n[0][2 * t] = n0v; sh.s_n[0][2 * t + 1] = n1v; mbar_arrive(&sh.nready); }   // nready phase 0 = n before chunk 0
    if (n_owner && p.n_states) {
      float* ns = p.n_states + ((size_t)bh * (NC + 1)) * FDQK;
      ns[2 * t] = n0v; ns[2 * t + 1] = n1v;
    }
    float* npart = reinterpret_cast<float*>(smem + F_OFF_NP);
    bool ok = true;
    for (int k = 0; k < NC && ok; ++k) {
      const float g = p.gbar[(size_t)bh * NC + k];
      // the score MMAs of this chunk have finished reading K: scale its rows in place
      ok = mbar_wait(&sh.kfull, k & 1, err, 331) && mbar_wait(&sh.sfull, k & 1, err, 332);
      if (!ok) break;
      // every thread has finished reading the previous chunk's partial sums (it arrived on nready after reading)
      if (use_n && !mbar_wait(&sh.nready, k & 1, err, 334)) { ok = false; break; }
      const float* sc = sh.s_scale[k & 1];
      const int lc = (t & 7) ^ ((t >> 3) & 7);   // logical 16-byte column chunk of this thread (rows t>>3 + 16u)
#pragma unroll
      for (int b = 0; b < 4; ++b) {
        float ns[8];
#pragma unroll
        for (int e = 0; e < 8; ++e) ns[e] = 0.f;
#pragma unroll
        for (int u = 0; u < 8; ++u) {
          const int row = (t >> 3) + 16 * u;
          const float s = sc[row];
          uint4* ptr = reinterpret_cast<uint4*>(smem + F_OFF_K + b * 16384 + row * 128 + (t & 7) * 16);
          uint4 v = *ptr;
          uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            __nv_bfloat162 h2 = *reinterpret_cast<__nv_bfloat162*>(&w[e]);
            const float lo = __low2float(h2) * s, hi = __high2float(h2) * s;
            ns[2 * e] += lo; ns[2 * e + 1] += hi;
            w[e] = pack_bf16(lo, hi);
          }
          *ptr = make_uint4(w[0], w[1], w[2], w[3]);
        }
        if (use_n) {
          float4* dst = reinterpret_cast<float4*>(npart + (t >> 3) * 256 + b * 64 + lc * 8);
          dst[0] = make_float4(ns[0], ns[1], ns[2], ns[3]);
          dst[1] = make_float4(ns[4], ns[5], ns[6], ns[7]);
        }
      }
      fence_proxy_async_smem();
      mbar_arrive(&sh.kscaled);
      if (use_n) {
        mbar_arrive(&sh.nsum);
        if (!mbar_wait(&sh.nsum, k & 1, err, 333)) { ok = false; break; }
        float c0 = 0.f, c1 = 0.f;
#pragma unroll
        for (int gq = 0; gq < 16; ++gq) { c0 += npart[gq * 256 + 2 * t]; c1 += npart[gq * 256 + 2 * t + 1]; }
        n0v = fmaf(g, n0v, c0); n1v = fmaf(g, n1v, c1);
        sh.s_n[(k + 1) & 1][2 * t] = n0v; sh.s_n[(k + 1) & 1][2 * t + 1] = n1v;
        mbar_arrive(&sh.nready);
        if (n_owner && p.n_states) {
          float* nsd = p.n_states + ((size_t)bh * (NC + 1) + k + 1) * FDQK;
          nsd[2 * t] = n0v; nsd[2 * t + 1] = n1v;
        }
      }
    }
    if (ok && n_owner && p.n_last) { p.n_last[(size_t)bh * FDQK + 2 * t] = n0v; p.n_last[(size_t)bh * FDQK + 2 * t + 1] = n1v; }
  } else {
    // =============================== state pass warps ===============================
    const int quarter = warp & 3, hcol = (warp - 14) >> 2;
    const int r = quarter * 32 + lane;                       // tensor-memory lane
    const uint32_t lane_base = (uint32_t)(quarter * 32) << 16;
    const bool elected = (warp == 14 && lane == 0);
    uint8_t* const cb = smem + F_OFF_C;
    bool ok = true;
    // pass index q = 0 is the initial state, q = k + 1 the state after chunk k
    for (int q = 0; q <= NC && ok; ++q) {
      const bool last = (q == NC);
      const float gnext = last ? 1.f : p.gbar[(size_t)bh * NC + q];   // decay of the chunk this state enters
      if (q > 0) {
        if (!mbar_wait(&sh.pfull, (q - 1) & 1, err, 341)) { ok = false; break; }
        tc_fence_after_sync();
        // the TMA store of the previous bf16 copy must have left the buffer before it is overwritten
        if (p.store_states && !mbar_wait(&sh.cstore, (q - 1) & 1, err, 342)) { ok = false; break; }
      }
#pragma unroll
      for (int mh = 0; mh < 2; ++mh) {
        const int d = mh * 128 + r;                           // state row
        const uint32_t ta = (mh ? tC1 : tC0) + lane_base + hcol * 64;
        uint8_t* rowp = cb + (d >> 6) * 16384 + hcol * 8192 + (d & 63) * 128;
#pragma unroll
        for (int q4 = 0; q4 < 4; ++q4) {
          uint32_t v[16];
          if (q == 0) {
            if (p.c_init) {
              const float4* src = reinterpret_cast<const float4*>(p.c_init + ((size_t)bh * FDQK + d) * p.DHHV + e0 + hcol * 64 + q4 * 16);
#pragma unroll
              for (int c = 0; c < 4; ++c) {
                const float4 x = src[c];
                v[4 * c] = __float_as_uint(x.x); v[4 * c + 1] = __float_as_uint(x.y);
                v[4 * c + 2] = __float_as_uint(x.z); v[4 * c + 3] = __float_as_uint(x.w);
              }
            } else {
#pragma unroll
              for (int c = 0; c < 16; ++c) v[c] = 0u;
            }
          } else {
            tmem_ld16(ta + q4 * 16, v);
            tmem_wait_ld();
          }
          // bf16 copy: 16 columns = two 16-byte chunks of the 64-column box row
          uint4 lo4, hi4;
          lo4.x = pack_bf16(__uint_as_float(v[0]), __uint_as_float(v[1])); lo4.y = pack_bf16(__uint_as_float(v[2]), __uint_as_float(v[3]));
          lo4.z = pack_bf16(__uint_as_float(v[4]), __uint_as_float(v[5])); lo4.w = pack_bf16(__uint_as_float(v[6]), __uint_as_float(v[7]));
          hi4.x = pack_bf16(__uint_as_float(v[8]), __uint_as_float(v[9])); hi4.y = pack_bf16(__uint_as_float(v[10]), __uint_as_float(v[11]));
          hi4.z = pack_bf16(__uint_as_float(v[12]), __uint_as_float(v[13])); hi4.w = pack_bf16(__uint_as_float(v[14]), __uint_as_float(v[15]));
          *reinterpret_cast<uint4*>(rowp + (((q4 * 2) ^ (d & 7)) << 4)) = lo4;
          *reinterpret_cast<uint4*>(rowp + (((q4 * 2 + 1) ^ (d & 7)) << 4)) = hi4;
          if (last) {
            if (p.c_last) {
              float4* dst = reinterpret_cast<float4*>(p.c_last + ((size_t)bh * FDQK + d) * p.DHHV + e0 + hcol * 64 + q4 * 16);
#pragma unroll
              for (int c = 0; c < 4; ++c)
                dst[c] = make_float4(__uint_as_float(v[4 * c]), __uint_as_float(v[4 * c + 1]), __uint_as_float(v[4 * c + 2]),
                                     __uint_as_float(v[4 * c + 3]));
            }
          } else {
#pragma unroll
            for (int c = 0; c < 16; ++c) v[c] = __float_as_uint(__uint_as_float(v[c]) * gnext);
            tmem_st16(ta + q4 * 16, v);
          }
        }
      }
      tmem_wait_st();
      fence_proxy_async_smem();
      tc_fence_before_sync();
      mbar_arrive(&sh.cready);
      if (elected && p.store_states) {
        if (!mbar_wait(&sh.cready, q & 1, err, 343)) { ok = false; break; }
        const int y = (bh * (NC + 1) + q) * FDQK;
#pragma unroll
        for (int d4 = 0; d4 < 4; ++d4) {
          tma_store_2d(&mapCs, cb + d4 * 16384, e0, y + 64 * d4);
          tma_store_2d(&mapCs, cb + d4 * 16384 + 8192, e0 + 64, y + 64 * d4);
        }
        tma_store_commit();
        tma_store_wait_read();
        mbar_arrive(&sh.cstore);
      }
    }
    if (elected) tma_store_wait_all();
  }
  tc_fence_before_sync();
  __syncthreads();
  if (warp == 1) tmem_dealloc(tmem, 512);
}

// ---- host side --------------------------------------------------------------------------------------------
bool sm100_fused_fw_supported(int B, int NH, int S, int DHQK, int DHHV, int L, int dtype) {
  if (!(dtype == MLSTM_BF16 && L == FL && S % FL == 0 && DHQK == FDQK && DHHV % 128 == 0 && DHHV <= 1024)) return false;
  // a persistent CTA per (batch, head, 128 columns): worthwhile only when these fill the GPU
  return (long long)B * NH * (DHHV / 128) >= 96;
}

int sm100_fused_fw(const void* q, const void* k, const void* v, const GateBuffers& gb, const float* c_initial,
                   const float* n_initial, void* h, float* n_out, void* c_states, float* n_states, float* c_last,
                   float* n_last, const ChunkwiseDims& d, cudaStream_t st) {
  PhaseScope ps(PH_PAR_FW, st);
  CUtensorMap mQ, mK, mV, mCs;
  const uint64_t rows = (uint64_t)d.B * d.NH * d.S;
  if (!sm100_host::make_map_bf16(&mQ, q, rows, d.DHQK, 128, 64) || !sm100_host::make_map_bf16(&mK, k, rows, d.DHQK, 128, 64) ||
      !sm100_host::make_map_bf16(&mV, v, rows, d.DHHV, 128, 64) ||
      !sm100_host::make_map_bf16(&mCs, c_states ? c_states : q, (uint64_t)d.B * d.NH * (d.NC + 1) * d.DHQK, d.DHHV, 64, 64))
    return MLSTM_ERR_CUDA;
  FusedParams fp{};
  fp.vecB = gb.vecB; fp.iota = gb.iota; fp.m_tok = gb.m_tok; fp.abar = gb.abar; fp.bbar = gb.bbar; fp.gbar = gb.gbar;
  fp.c_init = c_initial; fp.n_init = n_initial; fp.h = (__nv_bfloat16*)h; fp.n_out = n_out;
  fp.n_states = n_states; fp.c_last = c_last; fp.n_last = n_last; fp.store_states = c_states != nullptr;
  fp.S = d.S; fp.NC = d.NC; fp.DHHV = d.DHHV; fp.variant = d.variant; fp.eps = d.eps; fp.qk_scale = d.qk_scale;
  MLSTM_CUDA_CHECK(cudaFuncSetAttribute(fused_fw_sm100, cudaFuncAttributeMaxDynamicSharedMemorySize, F_SMEM));
  dim3 grid(d.DHHV / 128, d.B * d.NH);
  fused_fw_sm100<<<grid, F_THREADS, F_SMEM, st>>>(mQ, mK, mV, mCs, fp);
  MLSTM_LAUNCH_CHECK();
  return MLSTM_OK;
}

}  // namespace mlstm
