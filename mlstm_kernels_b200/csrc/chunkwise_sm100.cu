// tcgen05 / TMEM / TMA implementation of the chunkwise mLSTM kernels for B200 (sm_100a).
// bf16 or f16 operands, f32 accumulation in tensor memory, chunk size 128, head dims multiples of 8 (tiles of 128: a tile
// hanging over the edge of a head dim is zero-padded by TMA on the way in, masked or clipped on the way out).
//
//   rec_sm100<BWD>   inter-chunk recurrence (forward C_k, n_k; backward deltaC_k).  A CTA owns a 128 x 128 tile
//                    of the state for one (batch, head) and walks the chunks in order; per chunk one
//                    (gated left)^T x right contraction on the tensor cores into a double-buffered TMEM
//                    accumulator, decay + accumulate of the running state in registers, bf16 state store.
//                    mlstm_kernels/triton/chunkwise/xl_chunk/fw_kernel_recurrent.py:14-230, bw_kernel_recurrent.py:15-181
//   par_body         intra-chunk kernel (par_fw_sm100, par_bw_sm100) for H, deltaV, deltaK, deltaQ.  Per (batch, head, chunk, 128-wide output tile):
//                    score = A B^T (TMEM) -> gate matrix applied by the CUDA cores, bf16 result written back to
//                    TMEM and used as the A operand of score x X; the inter-chunk term A x state is accumulated
//                    into the same TMEM tile first and row-scaled in place.  The L x L gate matrix never
//                    leaves the SM.
//                    fw_kernel_parallel.py:14-289, bw_kernel_parallel_dV.py, bw_kernel_parallel_dK.py, bw_kernel_parallel_dQ.py
// Operands arrive by TMA (128-byte swizzle, no multicast) through mbarrier rings (four half-chunk stages in the recurrence, three stages in the intra-chunk kernels); one warp produces,
// one thread issues the MMAs, the remaining warps do the element-wise work.  Every wait is bounded.
#include "common.cuh"
#include "launch.cuh"
#include "sm100.cuh"

namespace mlstm {

using namespace sm100;

__device__ int g_sm100_status = 0;  // first error code raised by a bounded wait (0 = none)

constexpr int CL = 128;  // chunk length handled by these kernels

// =====================================================================================================
// Inter-chunk recurrence
// =====================================================================================================
struct RecParams {
  const float* lscale;  // per token: abar (fw) or bbar (bw)
  const float* rscale;  // per token: nullptr (fw) or 1/(den+eps) (bw)
  float lmul;           // 1 (fw) or qk_scale (bw)
  const float* gbar;    // (BNH, NC)
  const float* c_init;  // (BNH, DHQK, DHHV) f32 or nullptr
  const float* n_init;  // (BNH, DHQK) or nullptr
  void* c_states;           // (BNH, NC+1, DHQK, DHHV), 16-bit elements of the input type
  float* n_states;          // (BNH, NC+1, DHQK) or nullptr
  float* c_final;           // (BNH, DHQK, DHHV) f32 or nullptr
  float* n_final;
  int S, SP, NC, DHQK, DHHV;   // SP = NC * 128: slots per (batch, head) of the per-token scale vectors
  int bh0;                     // first (batch, head) unit of this launch (a launch may cover a sub-range of the units)
};

constexpr int REC_THREADS = 640;                 // warp 0 TMA, 1 MMA, 2..9 gate the left tile, 10..17 own the state, 18 stores it, 19 keeps n
constexpr int REC_HALF = 64;                     // tokens per ring stage: half a chunk
constexpr int REC_STAGE_BYTES = 32768;           // 64 tokens: left tile 16 KB + right tile 16 KB
constexpr int REC_NPART_BYTES = 2 * 32 * 128 * 4;   // double-buffered partial column sums of the gated left tile
constexpr int REC_OUT_BYTES = 2 * 32768;         // double-buffered bf16 state tile staged for the TMA store
// operand ring depth (two chunks in flight)
constexpr int rec_stages(bool) { return 4; }
constexpr int rec_smem_bytes(bool bwd) {
  return rec_stages(bwd) * REC_STAGE_BYTES + (bwd ? 0 : REC_NPART_BYTES) + REC_OUT_BYTES + 1024;
}

// One ring stage holds 64 tokens of the left and of the right operand (boxes of 64 rows x 64 columns, 8 KB each:
// left columns d0.., d0+64.., right columns e0.., e0+64..).  A chunk is two stages; the product of a chunk is
// accumulated over both before the state warps fold it in.  The ring is deeper than one chunk so that the load of
// chunk s+2 is already in flight while chunk s is being gated and multiplied.
// TN = columns of the state tile (128, or 64 for small problems: twice as many CTAs, so that a launch with few
// (batch, head) units still covers the GPU).
// F16: the 16-bit element type is IEEE half instead of bf16 (operands, gated tiles, stored states, outputs).
template <bool BWD, int TN, bool F16>
__global__ void __launch_bounds__(REC_THREADS, 1)
rec_sm100(const __grid_constant__ CUtensorMap mapL, const __grid_constant__ CUtensorMap mapR,
          const __grid_constant__ CUtensorMap mapS, RecParams p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  constexpr int REC_STAGES = rec_stages(BWD);
  __shared__ uint64_t bar_full[REC_STAGES], bar_empty[REC_STAGES], bar_scaled[REC_STAGES], bar_acc_full[2], bar_acc_free[2], bar_nsum[2], bar_nread[2], bar_out_full[2], bar_out_free[2];
  __shared__ uint32_t s_tmem;
  __shared__ int s_abort;   // set by the first wait of this CTA that runs out; every other wait polls it
  // per-row scale factors of the left tile, copied with the stage (backward: two factors per row)
  __shared__ __align__(16) float s_scale[REC_STAGES][REC_HALF], s_scale2[BWD ? REC_STAGES : 1][REC_HALF];
  __shared__ float s_g[8];          // decay of the chunk, ring of eight (outlives the operand ring)

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  // 1-D grid (no 65535 limit on batch x heads), state tiles of one (batch, head) next to each other
  static_assert(TN == 128 || TN == 64, "state tile width");
  constexpr int HC = TN / 2;   // columns each of the two state-warp groups owns
  // head dims need not be multiples of the tile: the last tile hangs over the edge, where loads read zeros (the
  // tensor maps know the true extents), plain accesses are masked and the state store is clipped
  const int n_et = (p.DHHV + TN - 1) / TN, n_dt = (p.DHQK + 127) / 128;
  const int et = blockIdx.x % n_et, dt = (blockIdx.x / n_et) % n_dt, bh = p.bh0 + blockIdx.x / (n_et * n_dt);
  const int e0 = et * TN, d0 = dt * 128;
  const int NC = p.NC, NH2 = 2 * p.NC;   // ring steps: two per chunk
  const bool do_n = (!BWD) && et == 0 && (p.n_states != nullptr || p.n_final != nullptr);

  if (tid == 0) {
    s_abort = 0;
    for (int s = 0; s < REC_STAGES; ++s) {
      mbar_init(&bar_full[s], 1); mbar_init(&bar_empty[s], 1); mbar_init(&bar_scaled[s], 256);
    }
    for (int s = 0; s < 2; ++s) {
      mbar_init(&bar_acc_full[s], 1); mbar_init(&bar_acc_free[s], 256); mbar_init(&bar_nsum[s], 256); mbar_init(&bar_nread[s], 1);
      mbar_init(&bar_out_full[s], 256); mbar_init(&bar_out_free[s], 1);
    }
    fence_barrier_init();
    tma_prefetch_desc(&mapL); tma_prefetch_desc(&mapR); tma_prefetch_desc(&mapS);
  }
  if (warp == 1) { tmem_alloc(&s_tmem, 256); tmem_relinquish(); }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem = s_tmem;

  if (warp == 0) {
    // ---------------- TMA producer ----------------
    // The per-row scale vectors travel with the stage (bulk copies on the same barrier).  The decay of a chunk is a
    // single float: the warp keeps the values of 32 consecutive steps in its lanes and fetches the next 32 a whole
    // block ahead, so no global-memory latency sits between a stage becoming free and the next issue.
    auto load_g = [&](int blk) -> float {
      const int s = blk * 32 + lane;
      return s < NC ? p.gbar[(size_t)bh * NC + (BWD ? NC - 1 - s : s)] : 0.f;
    };
    float g_blk = load_g(0), g_nxt = load_g(1);
    int issued = 0;
    for (int h = 0; h < NH2; ++h) {
      const int st = h % REC_STAGES, s = h >> 1;
      if ((h & 1) == 0) {
        if (s > 0 && (s & 31) == 0) { g_blk = g_nxt; g_nxt = load_g((s >> 5) + 1); }
        const float g = __shfl_sync(0xffffffffu, g_blk, s & 31);
        if (lane == 0) s_g[s & 7] = g;   // read two or more barrier hand-overs later (MMA commit -> state warps)
      }
      int ok = 1;
      if (lane == 0) ok = mbar_wait(&bar_empty[st], ((h / REC_STAGES) & 1) ^ 1, &s_abort, &g_sm100_status, 101) ? 1 : 0;
      ok = __shfl_sync(0xffffffffu, ok, 0);
      if (!ok) break;
      if (lane == 0) {
        const int ck = BWD ? NC - 1 - s : s;
        // token rows past the end of the sequence (ragged last chunk) arrive as zeros; their scale slots hold zeros
        const int y = ck * CL + (h & 1) * REC_HALF;          // first token of this half chunk inside the sequence
        const size_t slot0 = (size_t)bh * p.SP + y;
        uint8_t* sl = smem + st * REC_STAGE_BYTES;
        mbar_expect_tx(&bar_full[st], 16384 + TN * 128 + (BWD ? 2 : 1) * REC_HALF * 4);
        bulk_load(s_scale[st], p.lscale + slot0, REC_HALF * 4, &bar_full[st]);
        if (BWD) bulk_load(s_scale2[st], p.rscale + slot0, REC_HALF * 4, &bar_full[st]);
        tma_load_3d(sl, &mapL, &bar_full[st], d0, y, bh);
        tma_load_3d(sl + 8192, &mapL, &bar_full[st], d0 + 64, y, bh);
        tma_load_3d(sl + 16384, &mapR, &bar_full[st], e0, y, bh);
        if (TN == 128) tma_load_3d(sl + 24576, &mapR, &bar_full[st], e0 + 64, y, bh);
      }
      issued = h + 1;
    }
    if (lane == 0 && issued < NH2 && issued > 0) {  // error path: let the copies in flight land before the CTA retires
      for (int h = max(0, issued - REC_STAGES); h < issued; ++h)
        mbar_wait(&bar_full[h % REC_STAGES], (h / REC_STAGES) & 1, nullptr, nullptr, 0);
    }
  } else if (warp == 1) {
    // ---------------- MMA issuer ----------------
    if (lane == 0) {
      constexpr uint32_t idesc = umma_idesc_16(F16, 128, TN, 1, 1);
      for (int h = 0; h < NH2; ++h) {
        const int st = h % REC_STAGES, s = h >> 1, buf = s & 1;
        if (!mbar_wait(&bar_scaled[st], (h / REC_STAGES) & 1, &s_abort, &g_sm100_status, 102)) break;
        if ((h & 1) == 0 && !mbar_wait(&bar_acc_free[buf], ((s >> 1) & 1) ^ 1, &s_abort, &g_sm100_status, 103)) break;
        tc_fence_after_sync();
        const uint32_t sl = smem_u32(smem + st * REC_STAGE_BYTES), sr = sl + 16384;
#pragma unroll
        for (int kk = 0; kk < REC_HALF / 16; ++kk)
          umma_ss(tmem + buf * 128, umma_desc_sw128(sl + kk * 2048, 8192, 1024),
                  umma_desc_sw128(sr + kk * 2048, 8192, 1024), idesc, ((h & 1) || kk > 0) ? 1u : 0u);
        umma_commit(&bar_empty[st]);
        if (h & 1) umma_commit(&bar_acc_full[buf]);
      }
    }
  } else if (warp < 10) {
    // ---------------- gating warps: scale the rows of the left tile in place; column sums give n ----------------
    const int ct = tid - 64;                       // 0..255
    bool ok = true;
    float ns[2][8];
    for (int h = 0; h < NH2; ++h) {
      const int st = h % REC_STAGES, s = h >> 1, nb = s & 1;
      if (!mbar_wait(&bar_full[st], (h / REC_STAGES) & 1, &s_abort, &g_sm100_status, 105)) { ok = false; break; }
      // two 64-column boxes of 64 rows x 128 B, 128-byte swizzle: the scale depends on the row only
      uint8_t* sl = smem + st * REC_STAGE_BYTES;
      if ((h & 1) == 0) {
#pragma unroll
        for (int b = 0; b < 2; ++b)
#pragma unroll
          for (int e = 0; e < 8; ++e) ns[b][e] = 0.f;
      }
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        const int r = (ct >> 3) + 32 * (u & 1);
        float sc = s_scale[st][r] * p.lmul;
        if (BWD) sc *= s_scale2[st][r];
        uint4* ptr = reinterpret_cast<uint4*>(sl + (u >> 1) * 8192 + r * 128 + (ct & 7) * 16);
        uint4 v = *ptr;
        uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          float lo, hi;
          Pair16<F16>::unpack(w[e], lo, hi);
          lo *= sc; hi *= sc;
          ns[u >> 1][2 * e] += lo; ns[u >> 1][2 * e + 1] += hi;
          w[e] = Pair16<F16>::pack(lo, hi);
        }
        *ptr = make_uint4(w[0], w[1], w[2], w[3]);
      }
      float* npart = reinterpret_cast<float*>(smem + REC_STAGES * REC_STAGE_BYTES) + nb * (32 * 128);
      if (do_n && (h & 1)) {
        // the n warp has read the partial sums of chunk s - 2 out of this buffer
        if (s >= 2 && !mbar_wait(&bar_nread[nb], ((s >> 1) - 1) & 1, &s_abort, &g_sm100_status, 109)) { ok = false; break; }
        const int lc = (ct & 7) ^ ((ct >> 3) & 7);   // logical 16-byte column chunk behind the swizzle
#pragma unroll
        for (int b = 0; b < 2; ++b) {
          float4* dst = reinterpret_cast<float4*>(npart + (ct >> 3) * 128 + b * 64 + lc * 8);
          dst[0] = make_float4(ns[b][0], ns[b][1], ns[b][2], ns[b][3]);
          dst[1] = make_float4(ns[b][4], ns[b][5], ns[b][6], ns[b][7]);
        }
      }
      fence_proxy_async_smem();
      mbar_arrive(&bar_scaled[st]);
      if (do_n && (h & 1)) mbar_arrive(&bar_nsum[nb]);   // partial column sums of chunk s are complete (n warp)
    }
  } else if (warp == 18) {
    // ---------------- store warp: one TMA store per 64-column box of each staged state tile ----------------
    if (lane == 0 && p.c_states != nullptr) {
      uint8_t* stage_base = smem + REC_STAGES * REC_STAGE_BYTES + (BWD ? 0 : REC_NPART_BYTES);
      for (int n = 0; n <= NC; ++n) {
        const int ob = n & 1;
        if (!mbar_wait(&bar_out_full[ob], (n >> 1) & 1, &s_abort, &g_sm100_status, 108)) break;
        const int slot = BWD ? NC - n : n;
        const int z = bh * (NC + 1) + slot;
        tma_store_3d(&mapS, stage_base + ob * 32768, e0, d0, z);
        if (TN == 128 && e0 + 64 < p.DHHV) tma_store_3d(&mapS, stage_base + ob * 32768 + 16384, e0 + 64, d0, z);
        tma_store_commit();
        asm volatile("cp.async.bulk.wait_group.read 1;" ::: "memory");   // the previous tile has left its buffer
        if (n >= 1) mbar_arrive(&bar_out_free[ob ^ 1]);
      }
      tma_store_wait_all();   // all state tiles have been written before the CTA retires
    }
  } else if (warp == 19) {
    // ---------------- n warp: n_{s+1} = gbar n_s + column sums of the gated left tile (no tensor cores needed) ----
    // Four columns per lane; the 32 partial sums of a column are added in a fixed order, so the result does not
    // depend on scheduling.
    if (do_n) {
      float4 nv = make_float4(0.f, 0.f, 0.f, 0.f);
      const bool d_in = d0 + 4 * lane < p.DHQK;   // the lane's four rows exist (DHQK is a multiple of 8)
      if (p.n_init && d_in) nv = *reinterpret_cast<const float4*>(p.n_init + (size_t)bh * p.DHQK + d0 + 4 * lane);
      if (p.n_states != nullptr && d_in)
        *reinterpret_cast<float4*>(p.n_states + ((size_t)bh * (NC + 1)) * p.DHQK + d0 + 4 * lane) = nv;
      bool ok = true;
      for (int s = 0; s < NC; ++s) {
        const int nb = s & 1;
        if (!mbar_wait(&bar_nsum[nb], (s >> 1) & 1, &s_abort, &g_sm100_status, 106)) { ok = false; break; }
        const float4* np4 = reinterpret_cast<const float4*>(smem + REC_STAGES * REC_STAGE_BYTES) + nb * (32 * 32) + lane;
        float4 cs = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll 8
        for (int g = 0; g < 32; ++g) { const float4 v = np4[g * 32]; cs.x += v.x; cs.y += v.y; cs.z += v.z; cs.w += v.w; }
        __syncwarp();
        if (lane == 0) mbar_arrive(&bar_nread[nb]);
        const float g = s_g[s & 7];
        nv.x = fmaf(g, nv.x, cs.x); nv.y = fmaf(g, nv.y, cs.y); nv.z = fmaf(g, nv.z, cs.z); nv.w = fmaf(g, nv.w, cs.w);
        if (p.n_states != nullptr && d_in)
          *reinterpret_cast<float4*>(p.n_states + ((size_t)bh * (NC + 1) + s + 1) * p.DHQK + d0 + 4 * lane) = nv;
      }
      if (ok && p.n_final && d_in) *reinterpret_cast<float4*>(p.n_final + (size_t)bh * p.DHQK + d0 + 4 * lane) = nv;
    }
  } else {
    // ---------------- state warps: fold each chunk's product into the running state, store it ----------------
    const int quarter = warp & 3, half = (warp - 10) >> 2;
    const int row = quarter * 32 + lane;           // state row (d)
    const int d = d0 + row, ecol = e0 + half * HC;
    float C[HC];
    if (p.c_init) {
      const float4* src = reinterpret_cast<const float4*>(p.c_init + ((size_t)bh * p.DHQK + d) * p.DHHV + ecol);
#pragma unroll
      for (int c = 0; c < HC / 4; ++c) {
        float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
        if (d < p.DHQK && ecol + 4 * c < p.DHHV) v = src[c];
        C[4 * c] = v.x; C[4 * c + 1] = v.y; C[4 * c + 2] = v.z; C[4 * c + 3] = v.w;
      }
    } else {
#pragma unroll
      for (int c = 0; c < HC; ++c) C[c] = 0.f;
    }
    // The bf16 state tile goes to shared memory in the 128-byte-swizzled box layout and leaves with one TMA store
    // per 64-column box (coalesced, asynchronous); two staging buffers, one store group in flight.
    uint8_t* stage_base = smem + REC_STAGES * REC_STAGE_BYTES + (BWD ? 0 : REC_NPART_BYTES);
    int n_out = 0;   // tiles written so far
    auto store_c = [&]() -> bool {
      if (p.c_states == nullptr) return true;
      const int ob = n_out & 1;
      if (n_out >= 2 && !mbar_wait(&bar_out_free[ob], ((n_out >> 1) - 1) & 1, &s_abort, &g_sm100_status, 107)) return false;
      // TN = 128: each group fills its own 64-column box; TN = 64: the groups share one box (four 16-byte pieces each)
      uint8_t* rowp = stage_base + ob * 32768 + (TN == 128 ? half * 16384 : 0) + row * 128;
      const int piece0 = (TN == 128) ? 0 : half * 4;
#pragma unroll
      for (int c = 0; c < HC / 8; ++c) {
        uint4 v;
        v.x = Pair16<F16>::pack(C[8 * c], C[8 * c + 1]); v.y = Pair16<F16>::pack(C[8 * c + 2], C[8 * c + 3]);
        v.z = Pair16<F16>::pack(C[8 * c + 4], C[8 * c + 5]); v.w = Pair16<F16>::pack(C[8 * c + 6], C[8 * c + 7]);
        *reinterpret_cast<uint4*>(rowp + (((piece0 + c) ^ (row & 7)) << 4)) = v;
      }
      fence_proxy_async_smem();
      mbar_arrive(&bar_out_full[ob]);   // the store warp ships the tile
      ++n_out;
      return true;
    };
    bool ok = store_c();   // the state before the first step (slot 0 forward, slot NC backward)
    for (int s = 0; s < NC && ok; ++s) {
      const int buf = s & 1;
      if (!mbar_wait(&bar_acc_full[buf], (s >> 1) & 1, &s_abort, &g_sm100_status, 104)) { ok = false; break; }
      tc_fence_after_sync();
      const float g = s_g[s & 7];
      const uint32_t ta = tmem + ((uint32_t)(quarter * 32) << 16) + buf * 128 + half * HC;
#pragma unroll
      for (int q4 = 0; q4 < HC / 16; ++q4) {
        uint32_t rr[16];
        tmem_ld16(ta + q4 * 16, rr);
        tmem_wait_ld();
#pragma unroll
        for (int c = 0; c < 16; ++c) C[q4 * 16 + c] = fmaf(g, C[q4 * 16 + c], __uint_as_float(rr[c]));
      }
      tc_fence_before_sync();
      mbar_arrive(&bar_acc_free[buf]);
      ok = store_c();
    }
    if (ok && p.c_final) {
      float4* fd = reinterpret_cast<float4*>(p.c_final + ((size_t)bh * p.DHQK + d) * p.DHHV + ecol);
#pragma unroll
      for (int c = 0; c < HC / 4; ++c)
        if (d < p.DHQK && ecol + 4 * c < p.DHHV) fd[c] = make_float4(C[4 * c], C[4 * c + 1], C[4 * c + 2], C[4 * c + 3]);
    }
  }
  tc_fence_before_sync();
  __syncthreads();
  if (warp == 1) tmem_dealloc(tmem, 256);
}

// =====================================================================================================
// Intra-chunk kernel.  Output tile rows r = tokens of one chunk, 128 output columns.
//   out[r,:] = sum_c G[r,c] X[c,:] + rowscale_r * (A[r,:] . State)
//   G[r,c]   = gate(r,c) * (A[r,:] . B[c,:])
//   mode  A    B    contraction  gate   X    State operand                  rowscale            out
//   H     Q    K    DHQK         lower  V    C_k        [DHQK x DHHV]       s*bbar_r            H (divided by den)
//   DV    K    Q    DHQK         upper  dH   dC_{k+1}   [DHQK x DHHV]       abar_r              dV
//   DK    V    dH   DHHV         upper  Q    dC_{k+1}^T (rows d, cols e)    abar_r              dK
//   DQ    dH   V    DHHV         lower  K    C_k^T      (rows d, cols e)    s*bbar_r/(den_r+e)  dQ
// lower: c <= r, (i,j) = (r,c); upper: c >= r, (i,j) = (c,r);
// gate = s * exp((b_i - b_j) + iota_j - m_i) [* 1/(den_i+eps) in the three backward modes].
// grid (ceil(DO / 128 / PAR_MAXSUB), NC, B*NH), two CTAs per SM; 320 threads: warp 0 TMA, warp 1 MMA, warps 2..9
// element-wise (two warps per 32-row quarter of the tile, each owning two 32-column chunks).  One CTA produces up to
// PAR_MAXSUB neighbouring output tiles of its chunk and mode, one after the other, from a single score tile.
// Time line of a CTA's first tile (measured with time stamps at the benchmark size, two CTAs sharing an SM): first
// slices land after ~1.8 us, score complete ~3.3 us, gating until ~5 us with the inter-chunk product arriving
// underneath (~5.5 us), second product ~6.4 us, epilogue and stores until ~8.8 us; every further tile takes ~5.5 us.
// Within a tile the kernel is bound by this chain of dependent steps (the same kernel with every operand resident in
// L2 runs at the same speed); the forward kernel as a whole runs at the HBM copy bandwidth.
// =====================================================================================================
enum { PM_H = 0, PM_DV = 1, PM_DK = 2, PM_DQ = 3 };

struct ParParams {
  const float *vecB, *iota, *m_tok, *abar, *bbar, *inv_den;  // per token, f32
  const float* n_states;                                     // H only
  uint16_t *out_h, *out_dv, *out_dk, *out_dq;   // 16-bit elements of the input type
  float* n_out;               // H only
  float *rowdot_q, *rowdot_k; // sum_d q dq (from DQ), sum_d k dk (from DK); one partial per output tile: [DHQK/128][tokens]
  size_t nslots;              // B * NH * SP
  int S, SP, NC, DHQK, DHHV, variant;   // SP = NC * 128: slots per (batch, head) of the per-token gate vectors
  float eps, qk_scale;
  int bh0;                    // first (batch, head) unit of this launch
};

constexpr int PAR_THREADS = 320;  // warp 0 TMA, warp 1 MMA, warps 2..9 element-wise
constexpr int PAR_STAGE = 32768;  // two 16 KB boxes: (A, B) slice pair, (A, state) slice pair, or a 128 x 128 tile
constexpr int PAR_NST = 3;        // ring depth
constexpr int PAR_MAXSUB = 4;     // output tiles one CTA produces at most
constexpr int PAR_SMEM = PAR_NST * PAR_STAGE + 1024;

// Shared-memory control block of one intra-chunk CTA (the operand ring lives in dynamic shared memory).
struct ParShared {
  uint64_t bar_full[PAR_NST], bar_empty[PAR_NST], bar_qdone[PAR_NST], bar_sfull, bar_afull, bar_gated, bar_hfull, bar_accfree, bar_done, bar_dot,
      bar_pair[4], bar_out;
  uint32_t tmem;
  int abort;                       // set by the first wait of this CTA that runs out; every other wait polls it
  __align__(16) float s_colE[CL];  // per-column term of the gate exponent, base 2 (see par_body)
  __align__(16) float s_colF[CL];  // 2^(colE_c - colP of the column's 32-column block)
  float s_colP[4];                 // largest colE of each 32-column block
  float s_part[2][CL];           // per-row partial sums exchanged between the two warps of a row
  float s_qn[2][CL];
  float s_n[512];
};

// One body for the four modes; `mode` is uniform over the CTA, so every branch on it is uniform (a single copy of the
// code keeps the instruction cache warm when CTAs of different modes share an SM).
// Gate factor of element (r, c): 2^(rowE_r + colE_c), every positive factor folded into the exponent:
//   lower (H, DQ), valid c <= r:  rowE = (b_r - m_r) log2e + log2(s [/(den_r+eps)]),   colE = (iota_c - b_c) log2e
//   upper (DV, DK), valid c >= r: rowE = (iota_r - b_r) log2e + log2(s),               colE = (b_c - m_c) log2e - log2(den_c+eps)
// A 32 x 32 block off the diagonal is gated without a transcendental per element: with colP = the largest colE of
// the block's columns, 2^(rowE_r + colE_c) = 2^(rowE_r + colP) * 2^(colE_c - colP); the column factors (one ex2 per
// column and CTA) lie in (0, 1], and the row factor (one ex2 per row and block) cannot overflow because every
// element of an off-diagonal block is a valid gate entry, bounded by s / (den + eps).  Where a column factor
// underflows the exact value is below 2^-100 as well.  The diagonal block keeps the exact per-element form (its
// masked columns may carry arbitrarily large colE).  The special-function unit (16 results per clock and SM) was
// the limit of the gating phase before: the warps of the busiest row quarter share one SM sub-partition.
template <bool F16>
__device__ __forceinline__ void
par_body(const int mode, const CUtensorMap* mapA, const CUtensorMap* mapB, const CUtensorMap* mapX,
         const CUtensorMap* mapSt, const CUtensorMap* mapE, const ParParams& p,
         ParShared& sh, const int o_tile0, const int nsub, const int ck, const int bh) {
  const bool LOWER = (mode == PM_H || mode == PM_DQ);
  const bool ST_MN = (mode == PM_H || mode == PM_DV);  // state operand N-contiguous in shared memory
  const bool HAS_E = (mode == PM_DQ || mode == PM_DK);  // extra tile for the gate-gradient row sums
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int o00 = o_tile0 * 128;   // first output column of the CTA's first tile
  const int DI = (mode == PM_H || mode == PM_DV) ? p.DHQK : p.DHHV;   // contraction dim of the score product
  const int DO = (mode == PM_H || mode == PM_DV) ? p.DHHV : p.DHQK;   // output width
  const int NC = p.NC, ND = (DI + 63) / 64;   // slices of 64 columns; a last partial slice is padded with zeros by TMA
  const int y0 = ck * CL;                         // first token of the chunk inside its sequence
  const int valid = min(CL, p.S - y0);            // tokens of the chunk that exist (ragged last chunk: < 128)
  const size_t out_row0 = (size_t)bh * p.S + y0;  // first row of the chunk in the (B*NH*S)-row token tensors
  const bool use_n = (mode == PM_H) && p.variant != MLSTM_SIG_NONORM && p.n_states != nullptr;

  if (tid == 0) {
    sh.abort = 0;
    for (int s = 0; s < PAR_NST; ++s) {
      mbar_init(&sh.bar_full[s], 1); mbar_init(&sh.bar_empty[s], 1); mbar_init(&sh.bar_qdone[s], 8);
    }
    mbar_init(&sh.bar_sfull, 1); mbar_init(&sh.bar_afull, 1); mbar_init(&sh.bar_gated, 256); mbar_init(&sh.bar_hfull, 1); mbar_init(&sh.bar_dot, 256);
    for (int s = 0; s < 4; ++s) mbar_init(&sh.bar_pair[s], 64);
    mbar_init(&sh.bar_out, 256); mbar_init(&sh.bar_accfree, 256); mbar_init(&sh.bar_done, 256);
    fence_barrier_init();
    tma_prefetch_desc(mapA); tma_prefetch_desc(mapB); tma_prefetch_desc(mapX); tma_prefetch_desc(mapSt);
    if (HAS_E) tma_prefetch_desc(mapE);
  }
  if (warp == 1) { tmem_alloc(&sh.tmem, 256); tmem_relinquish(); }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem = sh.tmem;
  const uint32_t tS = tmem, tAcc = tmem + 128;
  // Ring loads, in order: ND (A, B) slice pairs for the score product, ND (A, state) slice pairs for the inter-chunk
  // product (A comes from L2 the second time), the X tile, the E tile.  The score is complete - and the element-wise
  // warps start gating - while the second group is still arriving.
  // A CTA produces `nsub` (1 .. PAR_MAXSUB) neighbouring 128-column output tiles of the same chunk and mode.  The
  // score tile and its gated form are the same for all of them, so every tile after the first only needs its own
  // state slices, X and E tiles: the gated tile stays in tensor memory, the accumulator is reused once the previous
  // tile's epilogue has read it.
  const int n0 = 2 * ND + 1 + (HAS_E ? 1 : 0);          // loads of the first tile
  const int n1 = ND + 1 + (HAS_E ? 1 : 0);              // loads of every further tile
  const int n_loads = n0 + (nsub - 1) * n1;
  enum { LK_SCORE = 0, LK_STATE = 1, LK_X = 2, LK_E = 3 };
  // kind of the load at position l of tile `sub` (no divisions: this runs on the load-issue path)
  auto load_kind = [&](int sub, int l, int& it) -> int {
    if (sub == 0 && l < ND) { it = l; return LK_SCORE; }
    const int ls = l - (sub == 0 ? ND : 0);
    if (ls < ND) { it = ls; return LK_STATE; }
    it = 0;
    return ls == ND ? LK_X : LK_E;
  };

  if (warp == 0) {
    // ---------------- TMA producer ----------------
    if (lane == 0) {
      const int slot = LOWER ? ck : ck + 1;
      const int sz = bh * (NC + 1) + slot;   // slab of the state tensor (one DHQK x DHHV matrix per chunk boundary)
      int issued = 0;
      // Per stage: uses handed back by an MMA commit so far (phase counter of bar_empty) and score pairs read for
      // q . n so far (phase counter of bar_qdone).  Scalars picked by comparisons, not arrays: a dynamically indexed
      // array would live in local memory, and with nearly all of L1 configured as shared memory every access to it
      // is a round trip to L2 on the load-issue path.
      int rm0 = 0, rm1 = 0, rm2 = 0, rq0 = 0, rq1 = 0, rq2 = 0;
      int st = 0, sub = 0, l = 0;                        // stage, tile and position inside the tile of load `ld`
      int pk1 = 0, pk2 = 0, pk3 = 0, ps1 = 0, ps2 = 0, ps3 = 0;   // kind and tile of the last three loads
      for (int ld = 0; ld < n_loads; ++ld) {
        int it;
        const int kind = load_kind(sub, l, it);
        if (ld >= PAR_NST) {   // the stage's previous occupant (three loads back) must be gone
          const int pkind = pk3, psub = ps3;
          bool okw;
          if (pkind == LK_SCORE || pkind == LK_STATE || (pkind == LK_X && HAS_E)) {
            const int rm = st == 0 ? rm0 : (st == 1 ? rm1 : rm2);
            okw = mbar_wait(&sh.bar_empty[st], (rm - 1) & 1, &sh.abort, &g_sm100_status, 201);
            // the element-wise warps read the A box of a score pair (q . n)
            if (okw && use_n && pkind == LK_SCORE) {
              const int rq = st == 0 ? rq0 : (st == 1 ? rq1 : rq2);
              okw = mbar_wait(&sh.bar_qdone[st], (rq - 1) & 1, &sh.abort, &g_sm100_status, 212);
            }
          } else {   // the staging buffer of a tile (its E stage, or its X stage in the modes without E) is handed
            okw = mbar_wait(&sh.bar_done, psub & 1, &sh.abort, &g_sm100_status, 215);   // back when the tile has been stored
          }
          if (!okw) break;
        }
        const int o0 = o00 + 128 * sub;
        uint8_t* sb = smem + st * PAR_STAGE;
        mbar_expect_tx(&sh.bar_full[st], PAR_STAGE);
        if (kind == LK_SCORE) {
          tma_load_3d(sb, mapA, &sh.bar_full[st], 64 * it, y0, bh);
          tma_load_3d(sb + 16384, mapB, &sh.bar_full[st], 64 * it, y0, bh);
        } else if (kind == LK_STATE) {
          tma_load_3d(sb, mapA, &sh.bar_full[st], 64 * it, y0, bh);
          if (ST_MN) {
            tma_load_3d(sb + 16384, mapSt, &sh.bar_full[st], o0, 64 * it, sz);
            tma_load_3d(sb + 16384 + 8192, mapSt, &sh.bar_full[st], o0 + 64, 64 * it, sz);
          } else {
            tma_load_3d(sb + 16384, mapSt, &sh.bar_full[st], 64 * it, o0, sz);
          }
        } else {
          const CUtensorMap* m = (kind == LK_X) ? mapX : mapE;
          tma_load_3d(sb, m, &sh.bar_full[st], o0, y0, bh);
          tma_load_3d(sb + 16384, m, &sh.bar_full[st], o0 + 64, y0, bh);
        }
        if (kind == LK_SCORE || kind == LK_STATE || (kind == LK_X && HAS_E)) { rm0 += (st == 0); rm1 += (st == 1); rm2 += (st == 2); }
        if (kind == LK_SCORE) { rq0 += (st == 0); rq1 += (st == 1); rq2 += (st == 2); }
        issued = ld + 1;
        pk3 = pk2; pk2 = pk1; pk1 = kind; ps3 = ps2; ps2 = ps1; ps1 = sub;
        st = st == PAR_NST - 1 ? 0 : st + 1;
        if (++l == (sub == 0 ? n0 : n1)) { l = 0; ++sub; }
      }
      if (issued < n_loads && issued > 0) {  // error path: let the copies in flight land before the CTA retires
        for (int ld = max(0, issued - PAR_NST); ld < issued; ++ld)
          mbar_wait(&sh.bar_full[ld % PAR_NST], (ld / PAR_NST) & 1, nullptr, nullptr, 0);
      }
    }
  } else if (warp == 1) {
    // ---------------- MMA issuer ----------------
    if (lane == 0) {
      constexpr uint32_t idesc_s = umma_idesc_16(F16, 128, 128, 0, 0);
      const uint32_t idesc_st = ST_MN ? umma_idesc_16(F16, 128, 128, 0, 1) : umma_idesc_16(F16, 128, 128, 0, 0);
      constexpr uint32_t idesc_x = umma_idesc_16(F16, 128, 128, 0, 1);
      bool ok = true;
      for (int ld = 0; ld < ND; ++ld) {            // score: S = A . B^T
        const int st = ld % PAR_NST;
        if (!mbar_wait(&sh.bar_full[st], (ld / PAR_NST) & 1, &sh.abort, &g_sm100_status, 202)) { ok = false; break; }
        tc_fence_after_sync();
        const uint32_t sa = smem_u32(smem + st * PAR_STAGE), sb = sa + 16384;
#pragma unroll
        for (int kk = 0; kk < 4; ++kk)
          umma_ss(tS, umma_desc_sw128(sa + kk * 32, 16, 1024), umma_desc_sw128(sb + kk * 32, 16, 1024), idesc_s,
                  (ld > 0 || kk > 0) ? 1u : 0u);
        umma_commit(&sh.bar_empty[st]);
      }
      if (ok) umma_commit(&sh.bar_sfull);
      for (int sub = 0; sub < nsub && ok; ++sub) {
        const int lbase = sub == 0 ? ND : n0 + (sub - 1) * n1;   // first state pair of this tile
        // the accumulator tile is free once the previous tile's epilogue has read it
        if (sub > 0 && !mbar_wait(&sh.bar_accfree, (sub - 1) & 1, &sh.abort, &g_sm100_status, 216)) { ok = false; break; }
        if (sub > 0) tc_fence_after_sync();
        for (int it = 0; it < ND; ++it) {           // inter-chunk term: Acc = A . State
          const int ld = lbase + it, st = ld % PAR_NST;
          if (!mbar_wait(&sh.bar_full[st], (ld / PAR_NST) & 1, &sh.abort, &g_sm100_status, 213)) { ok = false; break; }
          tc_fence_after_sync();
          const uint32_t sa = smem_u32(smem + st * PAR_STAGE), ss = sa + 16384;
#pragma unroll
          for (int kk = 0; kk < 4; ++kk) {
            const uint64_t bdesc = ST_MN ? umma_desc_sw128(ss + kk * 2048, 8192, 1024) : umma_desc_sw128(ss + kk * 32, 16, 1024);
            umma_ss(tAcc, umma_desc_sw128(sa + kk * 32, 16, 1024), bdesc, idesc_st, (it > 0 || kk > 0) ? 1u : 0u);
          }
          umma_commit(&sh.bar_empty[st]);
        }
        if (!ok) break;
        umma_commit(&sh.bar_afull);
        const int ldx = lbase + ND, stx = ldx % PAR_NST;
        ok = mbar_wait(&sh.bar_full[stx], (ldx / PAR_NST) & 1, &sh.abort, &g_sm100_status, 203) &&
             mbar_wait(&sh.bar_gated, sub & 1, &sh.abort, &g_sm100_status, 204);
        if (!ok) break;
        tc_fence_after_sync();
        const uint32_t sx = smem_u32(smem + stx * PAR_STAGE);
#pragma unroll
        for (int kk = 0; kk < 8; ++kk)
          umma_ts(tAcc, tS + kk * 8, umma_desc_sw128(sx + kk * 2048, 16384, 1024), idesc_x, 1u);
        if (HAS_E) umma_commit(&sh.bar_empty[stx]);   // the output is staged in the E stage: X's stage is free again
        umma_commit(&sh.bar_hfull);
      }
    }
  } else {
    // ---------------- element-wise warps: two warps per 32-row quarter, each owning two 32-column chunks ----
    const int quarter = warp & 3, half = (warp - 2) >> 2;
    const int r = quarter * 32 + lane;
    const size_t tok = (size_t)bh * p.SP + y0 + r;   // slot of this row in the per-token gate vectors
    const float b_r = p.vecB[tok], iota_r = p.iota[tok], m_r = p.m_tok[tok];
    const float inv_r = (mode == PM_H) ? 1.f : p.inv_den[tok];
    constexpr float kLog2e = 1.4426950408889634f;
    const float rowE = (LOWER ? (b_r - m_r) : (iota_r - b_r)) * kLog2e +
                       __log2f((mode == PM_DQ) ? p.qk_scale * inv_r : p.qk_scale);
    if (half == 0) {   // this thread's row in its role as a column of the gate matrix
      const float colE = LOWER ? (iota_r - b_r) * kLog2e : (b_r - m_r) * kLog2e + __log2f(inv_r);
      float colP = colE;
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) colP = fmaxf(colP, __shfl_xor_sync(0xffffffffu, colP, o));
      if (!(colP > -3.0e38f)) colP = 0.f;   // a block whose columns are all switched off
      sh.s_colE[r] = colE;
      sh.s_colF[r] = ex2_approx(colE - colP);
      if (lane == 0) sh.s_colP[quarter] = colP;
    }
    float rowscale;
    if (mode == PM_H) rowscale = p.qk_scale * p.bbar[tok];
    else if (mode == PM_DQ) rowscale = p.qk_scale * p.bbar[tok] * inv_r;
    else rowscale = p.abar[tok];
    if (use_n) {
      const float* nsrc = p.n_states + ((size_t)bh * (NC + 1) + ck) * p.DHQK;
      for (int dd = tid - 64; dd < ND * 64; dd += 256) sh.s_n[dd] = dd < p.DHQK ? nsrc[dd] : 0.f;   // zero padding
    }
    asm volatile("bar.sync 1, 256;" ::: "memory");  // gate vectors and n visible to the element-wise warps

    bool ok = true;
    // q . n_{k-1} for the denominator (H only): each thread reads half of its row of every Q slice from the
    // TMA stage (the stage is released to the producer only after these reads)
    float qn = 0.f;
    if (use_n) {
      for (int it = 0; it < ND && ok; ++it) {
        const int st = it % PAR_NST;
        if (!mbar_wait(&sh.bar_full[st], (it / PAR_NST) & 1, &sh.abort, &g_sm100_status, 207)) { ok = false; break; }
        const uint8_t* rowp = smem + st * PAR_STAGE + r * 128;
#pragma unroll
        for (int cc = 0; cc < 4; ++cc) {
          const int lc = half * 4 + cc;                      // logical 16-byte chunk of the 64-column slice
          const uint4 v = *reinterpret_cast<const uint4*>(rowp + ((lc ^ (r & 7)) << 4));
          const uint32_t w[4] = {v.x, v.y, v.z, v.w};
          const float* nn = sh.s_n + it * 64 + lc * 8;
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            float lo, hi;
            Pair16<F16>::unpack(w[e], lo, hi);
            qn = fmaf(lo, nn[2 * e], qn);
            qn = fmaf(hi, nn[2 * e + 1], qn);
          }
        }
        fence_proxy_async_smem();   // generic-proxy reads ordered before the TMA refill of the stage
        __syncwarp();
        if (lane == 0) mbar_arrive(&sh.bar_qdone[st]);
      }
      sh.s_qn[half][r] = qn;
    }

    const uint32_t lane_base = (uint32_t)(quarter * 32) << 16;
    float rowsum = 0.f;
    ok = ok && mbar_wait(&sh.bar_sfull, 0, &sh.abort, &g_sm100_status, 205);
    if (ok) {
      tc_fence_after_sync();
      // Tensor memory is read 16 columns at a time, the next load in flight while the current one is processed.
      // gate the score tile; the bf16 result goes back to tensor memory as the A operand of the second product.
      // Both warps of a quarter first read their chunks, then (after a warp-pair sync) write: the bf16 words of
      // chunk cq land on columns [16 cq, 16 cq + 16), which the partner warp may still have to read.
      uint32_t pk[2][16];
#pragma unroll
      for (int u = 0; u < 2; ++u) {
        const int cq = half + 2 * u;
        const int c0 = cq * 32;
        const bool skip = LOWER ? (cq > quarter) : (cq < quarter);
        if (skip) {
#pragma unroll
          for (int c = 0; c < 16; ++c) pk[u][c] = 0u;
        } else {
          const bool diag = (cq == quarter);   // only the diagonal chunk needs the causal mask
          uint32_t va[16], vb[16];
          tmem_ld16(tS + lane_base + c0, va);
          tmem_wait_ld(va);
          tmem_ld16(tS + lane_base + c0 + 16, vb);
#pragma unroll
          for (int hh = 0; hh < 2; ++hh) {
            if (hh == 1) tmem_wait_ld(vb);
            const uint32_t (&v)[16] = hh ? vb : va;
            if (diag) {
              const float4* ce = reinterpret_cast<const float4*>(sh.s_colE + c0 + 16 * hh);
#pragma unroll
              for (int c4 = 0; c4 < 4; ++c4) {
                const float4 e4 = ce[c4];
                const float ee[4] = {e4.x, e4.y, e4.z, e4.w};
                float g4[4];
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                  const int cl = 16 * hh + 4 * c4 + e;   // column inside the chunk; row inside the chunk is `lane`
                  float val = __uint_as_float(v[4 * c4 + e]) * ex2_approx(rowE + ee[e]);
                  if (LOWER ? (cl > lane) : (cl < lane)) val = 0.f;
                  g4[e] = val;
                  rowsum += val;
                }
                pk[u][8 * hh + 2 * c4] = Pair16<F16>::pack(g4[0], g4[1]);
                pk[u][8 * hh + 2 * c4 + 1] = Pair16<F16>::pack(g4[2], g4[3]);
              }
            } else {
              const float rf = ex2_approx(rowE + sh.s_colP[cq]);
              const float4* cf = reinterpret_cast<const float4*>(sh.s_colF + c0 + 16 * hh);
#pragma unroll
              for (int c4 = 0; c4 < 4; ++c4) {
                const float4 f4 = cf[c4];
                const float g0 = __uint_as_float(v[4 * c4]) * (rf * f4.x), g1 = __uint_as_float(v[4 * c4 + 1]) * (rf * f4.y);
                const float g2 = __uint_as_float(v[4 * c4 + 2]) * (rf * f4.z), g3 = __uint_as_float(v[4 * c4 + 3]) * (rf * f4.w);
                rowsum += (g0 + g1) + (g2 + g3);
                pk[u][8 * hh + 2 * c4] = Pair16<F16>::pack(g0, g1);
                pk[u][8 * hh + 2 * c4 + 1] = Pair16<F16>::pack(g2, g3);
              }
            }
          }
        }
      }
      // pair sync (bounded): both warps of the quarter have finished reading the score tile
      tc_fence_before_sync();
      mbar_arrive(&sh.bar_pair[quarter]);
      ok = mbar_wait(&sh.bar_pair[quarter], 0, &sh.abort, &g_sm100_status, 210);
      if (ok) {
        tc_fence_after_sync();
#pragma unroll
        for (int u = 0; u < 2; ++u) tmem_st16(tS + lane_base + (half + 2 * u) * 16, pk[u]);
        sh.s_part[half][r] = rowsum;
        tmem_wait_st();
      }
    }
    // ---- per output tile: row-scale the inter-chunk product, second product, epilogue, store ----
    float inv = 1.f;
    for (int sub = 0; sub < nsub && ok; ++sub) {
      const int o0 = o00 + 128 * sub;
      // the inter-chunk product of this tile has usually landed by now: row-scale it in place
      if (!mbar_wait(&sh.bar_afull, sub & 1, &sh.abort, &g_sm100_status, 214)) { ok = false; break; }
      tc_fence_after_sync();
#pragma unroll 1
      for (int cq = half; cq < 4; cq += 2) {
        uint32_t va[16], vb[16];
        const uint32_t ta = tAcc + lane_base + cq * 32;
        tmem_ld16(ta, va);
        tmem_wait_ld(va);
        tmem_ld16(ta + 16, vb);
#pragma unroll
        for (int c = 0; c < 16; ++c) va[c] = __float_as_uint(__uint_as_float(va[c]) * rowscale);
        tmem_wait_ld(vb);
        tmem_st16(ta, va);
#pragma unroll
        for (int c = 0; c < 16; ++c) vb[c] = __float_as_uint(__uint_as_float(vb[c]) * rowscale);
        tmem_st16(ta + 16, vb);
      }
      tmem_wait_st();
      tc_fence_before_sync();
      mbar_arrive(&sh.bar_gated);   // (first tile: the gated score tile is in place as well)
      if (!mbar_wait(&sh.bar_hfull, sub & 1, &sh.abort, &g_sm100_status, 206)) { ok = false; break; }
      tc_fence_after_sync();
      if (sub == 0 && mode == PM_H) {
        float den = 1.f;
        const float nn = (sh.s_part[0][r] + sh.s_part[1][r]) + rowscale * (use_n ? (sh.s_qn[0][r] + sh.s_qn[1][r]) : 0.f);
        if (p.variant == MLSTM_EXP) den = fmaxf(fabsf(nn), __expf(-m_r));
        else if (p.variant == MLSTM_SIG) den = fmaxf(fabsf(nn), 1.f);
        if (p.variant != MLSTM_SIG_NONORM) inv = 1.f / (den + p.eps);
        if (o_tile0 == 0 && half == 0 && r < valid) p.n_out[out_row0 + r] = den;
      }
      const int ldx = (sub == 0 ? 2 * ND : n0 + (sub - 1) * n1 + ND);    // ring index of this tile's X load; E follows it
      const uint8_t* erow = smem;
      if (HAS_E) {
        const int lde = ldx + 1, ste = lde % PAR_NST;
        if (!mbar_wait(&sh.bar_full[ste], (lde / PAR_NST) & 1, &sh.abort, &g_sm100_status, 208)) { ok = false; break; }
        erow = smem + ste * PAR_STAGE + r * 128;
      }
      float dot4[4] = {0.f, 0.f, 0.f, 0.f};   // four partial sums: no 64-long chain of dependent FMAs
      // The output tile is staged (bf16, two boxes of 128 rows x 128 bytes, 16-byte pieces XOR-swizzled by the row)
      // in the ring stage of the E tile - which arrives in exactly this layout, so a thread reads its E piece and
      // writes its output piece to the same 16 bytes - or, in the modes without E, in the stage the X tile occupied
      // (every MMA that read it has completed).  It is then written out by all element-wise warps together, each warp
      // instruction covering two full 256-byte rows of the tile.  Plain stores are posted, so the CTA retires without
      // waiting for them.
      uint8_t* ostage = smem + ((ldx + (HAS_E ? 1 : 0)) % PAR_NST) * PAR_STAGE;
#pragma unroll 1
      for (int cq = half; cq < 4; cq += 2) {
        uint32_t va[16], vb[16];
        const uint32_t ta = tAcc + lane_base + cq * 32;
        tmem_ld16(ta, va);
        tmem_wait_ld(va);
        tmem_ld16(ta + 16, vb);
        uint8_t* orow = ostage + (cq >> 1) * 16384 + r * 128;
#pragma unroll
        for (int c = 0; c < 4; ++c) {
          if (c == 2) tmem_wait_ld(vb);
          const uint32_t (&v)[16] = (c < 2) ? va : vb;
          float x[8];
#pragma unroll
          for (int e = 0; e < 8; ++e) x[e] = __uint_as_float(v[8 * (c & 1) + e]) * inv;
          const int sw = (((cq & 1) * 4 + c) ^ (r & 7)) << 4;   // 16-byte chunk (cq*4 + c) of the row, swizzled
          if (HAS_E) {
            const uint4 ev = *reinterpret_cast<const uint4*>(erow + (cq >> 1) * 16384 + sw);
            const uint32_t w[4] = {ev.x, ev.y, ev.z, ev.w};
#pragma unroll
            for (int e = 0; e < 4; ++e) {
              float lo, hi;
              Pair16<F16>::unpack(w[e], lo, hi);
              dot4[e] = fmaf(lo, x[2 * e], dot4[e]);
              dot4[e] = fmaf(hi, x[2 * e + 1], dot4[e]);
            }
          }
          uint4 o;
          o.x = Pair16<F16>::pack(x[0], x[1]); o.y = Pair16<F16>::pack(x[2], x[3]);
          o.z = Pair16<F16>::pack(x[4], x[5]); o.w = Pair16<F16>::pack(x[6], x[7]);
          *reinterpret_cast<uint4*>(orow + sw) = o;
        }
      }
      if (sub + 1 < nsub) {   // the accumulator tile may be overwritten by the next tile's inter-chunk product
        tc_fence_before_sync();
        mbar_arrive(&sh.bar_accfree);
      }
      const float dot = (dot4[0] + dot4[1]) + (dot4[2] + dot4[3]);
      mbar_arrive(&sh.bar_out);
      if (!mbar_wait(&sh.bar_out, sub & 1, &sh.abort, &g_sm100_status, 211)) { ok = false; break; }
      {
        uint16_t* outp = (mode == PM_H) ? p.out_h : (mode == PM_DV) ? p.out_dv : (mode == PM_DK) ? p.out_dk : p.out_dq;
        uint8_t* gbase = reinterpret_cast<uint8_t*>(outp + out_row0 * DO + o0);
        const int ew = warp - 2, j = lane & 15;          // 16-byte piece j of the 256-byte tile row
#pragma unroll
        for (int i2 = 0; i2 < 8; ++i2) {
          const int orow_i = 16 * i2 + 2 * ew + (lane >> 4);
          const uint4 o = *reinterpret_cast<const uint4*>(ostage + (j >> 3) * 16384 + orow_i * 128 + (((j & 7) ^ (orow_i & 7)) << 4));
          if (orow_i < valid && o0 + j * 8 < DO) *reinterpret_cast<uint4*>(gbase + (size_t)orow_i * DO * 2 + j * 16) = o;
        }
      }
      if (HAS_E) {
        sh.s_qn[half][r] = dot;
        mbar_arrive(&sh.bar_dot);
        if (half == 0) {
          if (!mbar_wait(&sh.bar_dot, sub & 1, &sh.abort, &g_sm100_status, 209)) { ok = false; break; }
          ((mode == PM_DQ) ? p.rowdot_q : p.rowdot_k)[(size_t)(o_tile0 + sub) * p.nslots + tok] = sh.s_qn[0][r] + sh.s_qn[1][r];
        }
      }
      if (sub + 1 < nsub) {
        // The staging stage of this tile may be refilled.  The TMA engine writes shared memory through the async
        // proxy: without this fence its data can be overtaken by this thread's own earlier (generic-proxy) staging
        // writes to the same addresses.
        fence_proxy_async_smem();
        mbar_arrive(&sh.bar_done);
      }
    }
  }
  tc_fence_before_sync();
  __syncthreads();
  if (warp == 1) tmem_dealloc(tmem, 256);
}

template <bool F16>
__global__ void __launch_bounds__(PAR_THREADS, 2)
par_fw_sm100(const __grid_constant__ CUtensorMap mQ, const __grid_constant__ CUtensorMap mK,
             const __grid_constant__ CUtensorMap mV, const __grid_constant__ CUtensorMap mC,
             const __grid_constant__ ParParams p) {
  __shared__ ParShared sh;
  const int T = (p.DHHV + 127) / 128;                 // output tiles per chunk; a CTA takes up to PAR_MAXSUB of them
  // 1-D grid in the order (tile group, chunk, batch x head): no 65535 limit on chunks or batch x heads
  const int gx = (T + PAR_MAXSUB - 1) / PAR_MAXSUB;
  const int x = blockIdx.x % gx, ck = (blockIdx.x / gx) % p.NC, bh = p.bh0 + blockIdx.x / (gx * p.NC);
  const int t0 = PAR_MAXSUB * x;
  par_body<F16>(PM_H, &mQ, &mK, &mV, &mC, &mV, p, sh, t0, min(PAR_MAXSUB, T - t0), ck, bh);
}

// deltaV, deltaK and deltaQ of one chunk in ONE launch: blockIdx.x enumerates the 128-wide output tiles of the three
// results, so the CTAs that read the same q, k, v, deltaH and state tiles of a chunk are scheduled next to each other
// and share them through L2 instead of re-reading them from HBM in three separate launches.
template <bool F16>
__global__ void __launch_bounds__(PAR_THREADS, 2)
par_bw_sm100(const __grid_constant__ CUtensorMap mQ, const __grid_constant__ CUtensorMap mK,
             const __grid_constant__ CUtensorMap mV, const __grid_constant__ CUtensorMap mDH,
             const __grid_constant__ CUtensorMap mC_k, const __grid_constant__ CUtensorMap mdC_mn,
             const __grid_constant__ CUtensorMap mdC_k,
             const __grid_constant__ ParParams p) {
  __shared__ ParShared sh;
  const int T_dv = (p.DHHV + 127) / 128, T_dk = (p.DHQK + 127) / 128;   // output tiles per chunk of dV, and of dK / dQ
  const int c_dv = (T_dv + PAR_MAXSUB - 1) / PAR_MAXSUB, c_dk = (T_dk + PAR_MAXSUB - 1) / PAR_MAXSUB;   // CTAs per mode
  const int gx = c_dv + 2 * c_dk;   // 1-D grid in the order (mode and tile group, chunk, batch x head)
  const int x = blockIdx.x % gx, ck = (blockIdx.x / gx) % p.NC, bh = p.bh0 + blockIdx.x / (gx * p.NC);
  int mode, pair, T;
  const CUtensorMap *a, *b, *xm, *stm, *e;
  if (x < c_dv) { mode = PM_DV; pair = x; T = T_dv; a = &mK; b = &mQ; xm = &mDH; stm = &mdC_mn; e = &mDH; }
  else if (x < c_dv + c_dk) { mode = PM_DK; pair = x - c_dv; T = T_dk; a = &mV; b = &mDH; xm = &mQ; stm = &mdC_k; e = &mK; }
  else { mode = PM_DQ; pair = x - c_dv - c_dk; T = T_dk; a = &mDH; b = &mV; xm = &mK; stm = &mC_k; e = &mQ; }
  par_body<F16>(mode, a, b, xm, stm, e, p, sh, PAR_MAXSUB * pair, min(PAR_MAXSUB, T - PAR_MAXSUB * pair), ck, bh);
}

// =====================================================================================================
// Host side
// =====================================================================================================
bool sm100_supported(int S, int DHQK, int DHHV, int L, int dtype) {
  // any sequence length: a ragged last chunk is handled by zero-filled loads and masked stores
  // head dims: multiples of 8 (16-byte rows for TMA and the vector stores); tiles that hang over the edge of a head
  // dim are padded with zeros by TMA on the way in and masked or clipped on the way out
  return (dtype == MLSTM_BF16 || dtype == MLSTM_F16) && L == CL && S >= 1 && DHQK % 8 == 0 && DHHV % 8 == 0 &&
         DHQK >= 8 && DHHV >= 8 && DHQK <= 512 && DHHV <= 1024;
}

// The kernels address token rows and state rows with 32-bit TMA coordinates and use 1-D grids: both row counts and
// every grid must stay below 2^31.
bool sm100_sizes_ok(int B, int NH, int S, int DHQK, int DHHV) {
  const uint64_t lim = 0x7fffffffull;
  const uint64_t bnh = (uint64_t)B * NH, nc = ((uint64_t)S + CL - 1) / CL;
  const uint64_t tiles = (uint64_t)((DHHV + 127) / 128 + 2 * ((DHQK + 127) / 128));
  return bnh * S < lim && bnh * (nc + 1) * DHQK < lim && bnh * nc * tiles < lim &&
         bnh * (uint64_t)((DHHV + 63) / 64) * ((DHQK + 127) / 128) < lim;
}

// cudaFuncSetAttribute once per kernel and device instead of on every call
template <typename K>
static int set_smem_once(K kern, int bytes, bool (&done)[64]) {
  int dev = 0;
  MLSTM_CUDA_CHECK(cudaGetDevice(&dev));
  if (dev < 0 || dev >= 64 || !done[dev]) {
    MLSTM_CUDA_CHECK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes));
    if (dev >= 0 && dev < 64) done[dev] = true;
  }
  return MLSTM_OK;
}

// Tensor maps depend only on (base pointer, rows, columns, box): a training loop calls with the same buffers over
// and over, so the last few encodings are kept per thread instead of calling the driver 3-7 times per launch.
struct MapKey { const void* base; uint64_t rows, cols, slabs; uint32_t box_rows, box_cols; bool f16; };
// slabs == 0: plain 2-D matrix [rows x cols]; otherwise a 3-D tensor [slabs x rows x cols]; f16: IEEE half, else bf16
static bool cached_map(CUtensorMap* m, const void* base, uint64_t rows, uint64_t cols, uint32_t box_rows,
                       uint32_t box_cols, uint64_t slabs, bool f16) {
  constexpr int N = 32;
  static thread_local MapKey keys[N];
  static thread_local CUtensorMap maps[N];
  static thread_local int used = 0, next = 0;
  for (int i = 0; i < used; ++i) {
    const MapKey& k = keys[i];
    if (k.base == base && k.rows == rows && k.cols == cols && k.slabs == slabs && k.box_rows == box_rows &&
        k.box_cols == box_cols && k.f16 == f16) {
      *m = maps[i];
      return true;
    }
  }
  const bool ok = slabs == 0 ? sm100_host::make_map_bf16(m, base, rows, cols, box_rows, box_cols, f16)
                             : sm100_host::make_map_bf16_3d(m, base, slabs, rows, cols, box_rows, box_cols, f16);
  if (!ok) return false;
  keys[next] = MapKey{base, rows, cols, slabs, box_rows, box_cols, f16};
  maps[next] = *m;
  next = (next + 1) % N;
  if (used < N) ++used;
  return true;
}

// token tensors (q, k, v, deltaH): one slab of S rows per (batch, head), so that a box hanging over the end of a
// sequence (ragged last chunk) reads zeros instead of the next head's tokens
static bool tok_map(CUtensorMap* m, const void* base, const ChunkwiseDims& d, int cols, int box_rows = 128) {
  return cached_map(m, base, (uint64_t)d.S, (uint64_t)cols, box_rows, 64, (uint64_t)d.B * d.NH, d.dtype == MLSTM_F16);
}
// per-chunk states: one slab of DHQK x DHHV per (batch, head, chunk boundary), so that a tile hanging over the edge of
// a head dim reads zeros (and is clipped on the way out) instead of touching the next slab
static bool state_map(CUtensorMap* m, const void* base, const ChunkwiseDims& d, int box_rows) {
  return cached_map(m, base, (uint64_t)d.DHQK, (uint64_t)d.DHHV, box_rows, 64, (uint64_t)d.B * d.NH * (d.NC + 1),
                    d.dtype == MLSTM_F16);
}

template <bool BWD, int TN, bool F16>
static int launch_rec_tn(const CUtensorMap& mL, const CUtensorMap& mR, const CUtensorMap& mS, const RecParams& rp,
                         const ChunkwiseDims& d, int units, cudaStream_t st) {
  auto kern = rec_sm100<BWD, TN, F16>;
  static bool attr_done[64] = {};
  if (int rc = set_smem_once(kern, rec_smem_bytes(BWD), attr_done)) return rc;
  const unsigned grid = (unsigned)((d.DHHV + TN - 1) / TN) * (unsigned)((d.DHQK + 127) / 128) * (unsigned)units;
  kern<<<grid, REC_THREADS, rec_smem_bytes(BWD), st>>>(mL, mR, mS, rp);
  MLSTM_LAUNCH_CHECK();
  return MLSTM_OK;
}

// number of SMs of the current device (queried once per device)
static int sm_count() {
  static int cached[64] = {};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 148;
  if (cached[dev] == 0) {
    int n = 0;
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 148;
    cached[dev] = n;
  }
  return cached[dev];
}

long sm100_recurrence_ctas(const ChunkwiseDims& d) {
  return (long)((d.DHHV + 127) / 128) * ((d.DHQK + 127) / 128) * d.B * d.NH;
}
int sm100_sm_count() { return sm_count(); }

template <bool BWD>
static int launch_rec(const void* left, const void* right, RecParams rp, const ChunkwiseDims& d, UnitRange ur,
                      cudaStream_t st) {
  rp.bh0 = ur.first;
  const int units = ur.count < 0 ? d.B * d.NH - ur.first : ur.count;
  if (units <= 0) return MLSTM_OK;
  CUtensorMap mL, mR, mS;
  // recurrence operands arrive in half-chunk boxes (64 tokens x 64 columns)
  if (!tok_map(&mL, left, d, d.DHQK, REC_HALF) || !tok_map(&mR, right, d, d.DHHV, REC_HALF)) return MLSTM_ERR_CUDA;
  // store map over the per-chunk states; when no states are wanted (segment summary) the map is never used
  if (!state_map(&mS, rp.c_states ? (const void*)rp.c_states : left, d, 128)) return MLSTM_ERR_CUDA;
  // One CTA per SM walks all chunks of its state tile.  With 128-column tiles a launch of few (batch, head) units
  // leaves SMs idle; 64-column tiles double the CTAs as long as they still fit one wave.
  const long ctas128 = sm100_recurrence_ctas(d);
  const bool f16 = d.dtype == MLSTM_F16;
  if (2 * ctas128 <= sm_count())
    return f16 ? launch_rec_tn<BWD, 64, true>(mL, mR, mS, rp, d, units, st) : launch_rec_tn<BWD, 64, false>(mL, mR, mS, rp, d, units, st);
  return f16 ? launch_rec_tn<BWD, 128, true>(mL, mR, mS, rp, d, units, st) : launch_rec_tn<BWD, 128, false>(mL, mR, mS, rp, d, units, st);
}

int sm100_recurrent_fw(const void* k, const void* v, const GateBuffers& gb, const float* c_initial,
                       const float* n_initial, void* c_states, float* n_states, float* c_last, float* n_last,
                       const ChunkwiseDims& d, cudaStream_t st, UnitRange ur) {
  PhaseScope ps(PH_REC_FW, st);
  RecParams rp{gb.abar, nullptr, 1.f, gb.gbar, c_initial, n_initial, c_states,
               d.variant == MLSTM_SIG_NONORM ? nullptr : n_states, c_last, d.variant == MLSTM_SIG_NONORM ? nullptr : n_last, d.S, d.SP, d.NC, d.DHQK, d.DHHV, 0};
  return launch_rec<false>(k, v, rp, d, ur, st);
}

int sm100_recurrent_bw(const void* q, const void* dh, const GateBuffers& gb, const float* dc_last, void* dc_states,
                       float* dc_initial, const ChunkwiseDims& d, cudaStream_t st, UnitRange ur) {
  PhaseScope ps(PH_REC_BW, st);
  RecParams rp{gb.bbar, gb.inv_den, d.qk_scale, gb.gbar, dc_last, nullptr, dc_states, nullptr,
               dc_initial, nullptr, d.S, d.SP, d.NC, d.DHQK, d.DHHV, 0};
  return launch_rec<true>(q, dh, rp, d, ur, st);
}

static ParParams base_params(const GateBuffers& gb, const ChunkwiseDims& d) {
  ParParams pp{};
  pp.vecB = gb.vecB; pp.iota = gb.iota; pp.m_tok = gb.m_tok; pp.abar = gb.abar; pp.bbar = gb.bbar;
  pp.inv_den = gb.inv_den;
  pp.nslots = (size_t)d.B * d.NH * d.SP;
  pp.S = d.S; pp.SP = d.SP; pp.NC = d.NC; pp.DHQK = d.DHQK; pp.DHHV = d.DHHV; pp.variant = d.variant; pp.eps = d.eps;
  pp.qk_scale = d.qk_scale;
  return pp;
}

int sm100_parallel_fw(const void* q, const void* k, const void* v, const GateBuffers& gb, const void* c_states,
                      const float* n_states, void* h, float* n_out, const ChunkwiseDims& d, cudaStream_t st,
                      UnitRange ur) {
  const int units = ur.count < 0 ? d.B * d.NH - ur.first : ur.count;
  if (units <= 0) return MLSTM_OK;
  PhaseScope ps(PH_PAR_FW, st);
  CUtensorMap mQ, mK, mV, mC;
  if (!tok_map(&mQ, q, d, d.DHQK) || !tok_map(&mK, k, d, d.DHQK) || !tok_map(&mV, v, d, d.DHHV) ||
      !state_map(&mC, c_states, d, 64))
    return MLSTM_ERR_CUDA;
  ParParams pp = base_params(gb, d);
  pp.n_states = n_states; pp.out_h = (uint16_t*)h; pp.n_out = n_out;
  pp.bh0 = ur.first;
  const bool f16 = d.dtype == MLSTM_F16;
  static bool attr_done[2][64] = {};
  if (int rc = f16 ? set_smem_once(par_fw_sm100<true>, PAR_SMEM, attr_done[1])
                   : set_smem_once(par_fw_sm100<false>, PAR_SMEM, attr_done[0])) return rc;
  // up to PAR_MAXSUB output tiles per CTA
  const unsigned grid = (unsigned)(((d.DHHV + 127) / 128 + PAR_MAXSUB - 1) / PAR_MAXSUB) * (unsigned)d.NC * (unsigned)units;
  if (f16) par_fw_sm100<true><<<grid, PAR_THREADS, PAR_SMEM, st>>>(mQ, mK, mV, mC, pp);
  else par_fw_sm100<false><<<grid, PAR_THREADS, PAR_SMEM, st>>>(mQ, mK, mV, mC, pp);
  MLSTM_LAUNCH_CHECK();
  return MLSTM_OK;
}

int sm100_parallel_bw(const void* q, const void* k, const void* v, const void* dh, const GateBuffers& gb,
                      const void* c_states, const void* dc_states, void* dq, void* dk, void* dv, float* qdq_parts,
                      float* kdk_parts, const ChunkwiseDims& d, cudaStream_t st, UnitRange ur) {
  const int units = ur.count < 0 ? d.B * d.NH - ur.first : ur.count;
  if (units <= 0) return MLSTM_OK;
  PhaseScope ps(PH_PAR_BW, st);
  CUtensorMap mQ, mK, mV, mDH, mC_k, mdC_mn, mdC_k;
  if (!tok_map(&mQ, q, d, d.DHQK) || !tok_map(&mK, k, d, d.DHQK) || !tok_map(&mV, v, d, d.DHHV) ||
      !tok_map(&mDH, dh, d, d.DHHV) || !state_map(&mC_k, c_states, d, 128) || !state_map(&mdC_mn, dc_states, d, 64) ||
      !state_map(&mdC_k, dc_states, d, 128))
    return MLSTM_ERR_CUDA;
  ParParams pp = base_params(gb, d);
  pp.out_dv = (uint16_t*)dv; pp.out_dk = (uint16_t*)dk; pp.out_dq = (uint16_t*)dq;
  pp.rowdot_q = qdq_parts; pp.rowdot_k = kdk_parts;
  pp.bh0 = ur.first;
  const bool f16 = d.dtype == MLSTM_F16;
  static bool attr_done[2][64] = {};
  if (int rc = f16 ? set_smem_once(par_bw_sm100<true>, PAR_SMEM, attr_done[1])
                   : set_smem_once(par_bw_sm100<false>, PAR_SMEM, attr_done[0])) return rc;
  // up to PAR_MAXSUB output tiles per CTA
  const unsigned grid = (unsigned)(((d.DHHV + 127) / 128 + PAR_MAXSUB - 1) / PAR_MAXSUB +
                                   2 * (((d.DHQK + 127) / 128 + PAR_MAXSUB - 1) / PAR_MAXSUB)) *
                        (unsigned)d.NC * (unsigned)units;
  if (f16) par_bw_sm100<true><<<grid, PAR_THREADS, PAR_SMEM, st>>>(mQ, mK, mV, mDH, mC_k, mdC_mn, mdC_k, pp);
  else par_bw_sm100<false><<<grid, PAR_THREADS, PAR_SMEM, st>>>(mQ, mK, mV, mDH, mC_k, mdC_mn, mdC_k, pp);
  MLSTM_LAUNCH_CHECK();
  return MLSTM_OK;
}

// Self-test of the bounded wait: one thread waits, for at most `limit` polls, on an mbarrier that nothing arrives
// at.  No copy is in flight and no tensor memory is held, so giving up is all that happens: the wait records
// `code` in the status word and the kernel returns.
__global__ void wait_expiry_selftest_kernel(uint32_t limit, int code) {
  __shared__ uint64_t bar;
  __shared__ int abort_flag;
  if (threadIdx.x == 0) {
    abort_flag = 0;
    mbar_init(&bar, 1);
    fence_barrier_init();
    mbar_wait(&bar, 0, &abort_flag, &g_sm100_status, code, limit);
  }
}

int sm100_wait_expiry_selftest(unsigned limit, int code, cudaStream_t st) {
  if (limit == 0 || limit > 1000000u || code <= 0) return MLSTM_ERR_UNSUPPORTED;   // a few milliseconds at most
  wait_expiry_selftest_kernel<<<1, 32, 0, st>>>(limit, code);
  MLSTM_LAUNCH_CHECK();
  return MLSTM_OK;
}

int sm100_force_load() {
  cudaFuncAttributes a;
  MLSTM_CUDA_CHECK(cudaFuncGetAttributes(&a, (rec_sm100<false, 128, false>)));
  MLSTM_CUDA_CHECK(cudaFuncGetAttributes(&a, (rec_sm100<false, 64, false>)));
  MLSTM_CUDA_CHECK(cudaFuncGetAttributes(&a, par_fw_sm100<false>));
  MLSTM_CUDA_CHECK(cudaFuncGetAttributes(&a, (rec_sm100<false, 128, true>)));
  MLSTM_CUDA_CHECK(cudaFuncGetAttributes(&a, (rec_sm100<false, 64, true>)));
  MLSTM_CUDA_CHECK(cudaFuncGetAttributes(&a, par_fw_sm100<true>));
  return MLSTM_OK;
}

// Reads (and optionally clears) the status word the bounded waits write on a timeout.  Synchronises the device.
int sm100_device_status(int reset, int* status) {
  MLSTM_CUDA_CHECK(cudaDeviceSynchronize());
  MLSTM_CUDA_CHECK(cudaMemcpyFromSymbol(status, g_sm100_status, sizeof(int)));
  if (reset) {
    const int zero = 0;
    MLSTM_CUDA_CHECK(cudaMemcpyToSymbol(g_sm100_status, &zero, sizeof(int)));
  }
  return MLSTM_OK;
}

}  // namespace mlstm
