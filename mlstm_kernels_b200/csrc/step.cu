// Recurrent decode step (HBM-bound): streams the f32 state C once in and once out with 128-bit
// accesses, keeps everything else on chip.
//
//   m' = max(logsigmoid(f) + m, i);  fbar = exp(logsigmoid(f) + m - m');  ibar = exp(i - m')
//   C' = fbar C + ibar k v^T;  n' = fbar n + ibar k;  h = (s q) C' / (max(|s q . n'|, exp(-m')) + eps)
// mlstm_kernels/triton/recurrent/fw_step_fused.py:19-195, mlstm_kernels/torch/recurrent/native_step.py:8-101.
//
// One CTA owns all DHQK rows of a TV-wide column slice of one (batch, head): the q.C' reduction is
// local to the CTA; q.n' is recomputed per CTA (DHQK values, negligible).
#include "common.cuh"
#include "launch.cuh"

namespace mlstm {

constexpr int STEP_THREADS = 256;
constexpr int STEP_TV = 64;              // columns per CTA
constexpr int STEP_CG = STEP_TV / 4;     // threads across the columns (float4 each)
constexpr int STEP_RG = STEP_THREADS / STEP_CG;  // row groups

template <typename TS> struct Vec4;
template <> struct Vec4<float> {
  static __device__ __forceinline__ float4 load(const float* p) { return __ldcs(reinterpret_cast<const float4*>(p)); }
  static __device__ __forceinline__ void store(float* p, float4 v) { __stcs(reinterpret_cast<float4*>(p), v); }
};
template <> struct Vec4<__nv_bfloat16> {
  static __device__ __forceinline__ float4 load(const __nv_bfloat16* p) {
    uint2 raw = __ldcs(reinterpret_cast<const uint2*>(p));
    __nv_bfloat162 a = *reinterpret_cast<__nv_bfloat162*>(&raw.x), b = *reinterpret_cast<__nv_bfloat162*>(&raw.y);
    return make_float4(__low2float(a), __high2float(a), __low2float(b), __high2float(b));
  }
  static __device__ __forceinline__ void store(__nv_bfloat16* p, float4 v) {
    __nv_bfloat162 a = __floats2bfloat162_rn(v.x, v.y), b = __floats2bfloat162_rn(v.z, v.w);
    uint2 raw;
    raw.x = *reinterpret_cast<uint32_t*>(&a);
    raw.y = *reinterpret_cast<uint32_t*>(&b);
    __stcs(reinterpret_cast<uint2*>(p), raw);
  }
};

// The gate pre-activations keep their own element type (f32 gates next to bf16 q, k, v is the usual set-up) and are
// widened to f32 before any arithmetic, as the reference does (fw_step_fused.py:88-94).
__device__ __forceinline__ float load_gate(const void* p, size_t idx, int gate_dtype) {
  if (gate_dtype == MLSTM_F32) return static_cast<const float*>(p)[idx];
  if (gate_dtype == MLSTM_BF16) return __bfloat162float(static_cast<const __nv_bfloat16*>(p)[idx]);
  return __half2float(static_cast<const __half*>(p)[idx]);
}

template <typename T, typename TS>
__global__ void __launch_bounds__(STEP_THREADS)
step_kernel(const T* __restrict__ q, const T* __restrict__ k, const T* __restrict__ v, const void* __restrict__ gi,
            const void* __restrict__ gf, int gate_dtype, const TS* __restrict__ c, const TS* __restrict__ n,
            const TS* __restrict__ m, T* __restrict__ h, TS* __restrict__ c_new, TS* __restrict__ n_new,
            TS* __restrict__ m_new, int DHQK, int DHHV, float eps) {
  extern __shared__ float sm[];
  float* s_q = sm;             // [DHQK] scaled q
  float* s_k = s_q + DHQK;     // [DHQK] ibar * k
  float* s_red = s_k + DHQK;   // [STEP_RG][STEP_TV] partial h, then reused
  __shared__ float s_warp[STEP_THREADS / 32];
  __shared__ float s_den;

  const int tid = threadIdx.x;
  // 1-D grid (no 65535 limit on batch x heads): the column tiles of one (batch, head) next to each other
  const int ntile = (DHHV + STEP_TV - 1) / STEP_TV;
  const int bh = blockIdx.x / ntile, tile = blockIdx.x % ntile, e0 = tile * STEP_TV;
  const int cgi = tid % STEP_CG, rg = tid / STEP_CG;
  const int e = e0 + cgi * 4;

  const float lf = logsigmoid_f(load_gate(gf, bh, gate_dtype));
  const float iv = load_gate(gi, bh, gate_dtype);
  const float m_old = to_f32(m[bh]);
  const float m_n = fmaxf(lf + m_old, iv);
  const float fbar = expf(lf + m_old - m_n);
  const float ibar = expf(iv - m_n);
  const float scale = rsqrtf((float)DHQK);

  // q, k into shared memory; q.n' partial
  float qn = 0.f;
  for (int d = tid; d < DHQK; d += STEP_THREADS) {
    const float qs = to_f32(q[(size_t)bh * DHQK + d]) * scale;
    const float ik = ibar * to_f32(k[(size_t)bh * DHQK + d]);
    const float nn = fmaf(fbar, to_f32(n[(size_t)bh * DHQK + d]), ik);
    s_q[d] = qs;
    s_k[d] = ik;
    qn = fmaf(qs, nn, qn);
    if (tile == 0) n_new[(size_t)bh * DHQK + d] = from_f32<TS>(nn);
  }
  qn = warp_sum(qn);
  if ((tid & 31) == 0) s_warp[tid >> 5] = qn;
  __syncthreads();
  if (tid == 0) {
    float t = 0.f;
    for (int w = 0; w < STEP_THREADS / 32; ++w) t += s_warp[w];
    s_den = fmaxf(fabsf(t), expf(-m_n)) + eps;
    if (tile == 0) m_new[bh] = from_f32<TS>(m_n);
  }

  float4 hv = make_float4(0.f, 0.f, 0.f, 0.f);
  if (e < DHHV) {
    const float4 vv = make_float4(to_f32(v[(size_t)bh * DHHV + e]), to_f32(v[(size_t)bh * DHHV + e + 1]),
                                  to_f32(v[(size_t)bh * DHHV + e + 2]), to_f32(v[(size_t)bh * DHHV + e + 3]));
    const TS* cp = c + (size_t)bh * DHQK * DHHV + e;
    TS* cn = c_new + (size_t)bh * DHQK * DHHV + e;
    constexpr int UNR = 8;
    int d = rg;
    for (; d + (UNR - 1) * STEP_RG < DHQK; d += UNR * STEP_RG) {
      float4 cv[UNR];
#pragma unroll
      for (int u = 0; u < UNR; ++u) cv[u] = Vec4<TS>::load(cp + (size_t)(d + u * STEP_RG) * DHHV);
#pragma unroll
      for (int u = 0; u < UNR; ++u) {
        const float kk = s_k[d + u * STEP_RG], qq = s_q[d + u * STEP_RG];
        float4 o;
        o.x = fmaf(fbar, cv[u].x, kk * vv.x);
        o.y = fmaf(fbar, cv[u].y, kk * vv.y);
        o.z = fmaf(fbar, cv[u].z, kk * vv.z);
        o.w = fmaf(fbar, cv[u].w, kk * vv.w);
        Vec4<TS>::store(cn + (size_t)(d + u * STEP_RG) * DHHV, o);
        hv.x = fmaf(qq, o.x, hv.x); hv.y = fmaf(qq, o.y, hv.y);
        hv.z = fmaf(qq, o.z, hv.z); hv.w = fmaf(qq, o.w, hv.w);
      }
    }
    for (; d < DHQK; d += STEP_RG) {
      const float4 cv = Vec4<TS>::load(cp + (size_t)d * DHHV);
      const float kk = s_k[d], qq = s_q[d];
      float4 o;
      o.x = fmaf(fbar, cv.x, kk * vv.x);
      o.y = fmaf(fbar, cv.y, kk * vv.y);
      o.z = fmaf(fbar, cv.z, kk * vv.z);
      o.w = fmaf(fbar, cv.w, kk * vv.w);
      Vec4<TS>::store(cn + (size_t)d * DHHV, o);
      hv.x = fmaf(qq, o.x, hv.x); hv.y = fmaf(qq, o.y, hv.y);
      hv.z = fmaf(qq, o.z, hv.z); hv.w = fmaf(qq, o.w, hv.w);
    }
  }
  // reduce the column partials over the row groups: first inside the warp (a warp spans 2 row groups)
  hv.x += __shfl_xor_sync(0xffffffffu, hv.x, 16);
  hv.y += __shfl_xor_sync(0xffffffffu, hv.y, 16);
  hv.z += __shfl_xor_sync(0xffffffffu, hv.z, 16);
  hv.w += __shfl_xor_sync(0xffffffffu, hv.w, 16);
  if ((tid & 31) < 16) {
    float* dst = s_red + (tid >> 5) * STEP_TV + cgi * 4;
    dst[0] = hv.x; dst[1] = hv.y; dst[2] = hv.z; dst[3] = hv.w;
  }
  __syncthreads();
  if (tid < STEP_TV && e0 + tid < DHHV) {
    float t = 0.f;
#pragma unroll
    for (int w = 0; w < STEP_THREADS / 32; ++w) t += s_red[w * STEP_TV + tid];
    h[(size_t)bh * DHHV + e0 + tid] = from_f32<T>(t / s_den);
  }
}

// T tokens in one launch, C slice resident in registers.  ROWS = rows of C per thread.
template <typename T, int ROWS>
__global__ void __launch_bounds__(STEP_THREADS)
step_sequence_kernel(const T* __restrict__ q, const T* __restrict__ k, const T* __restrict__ v,
                     const void* __restrict__ gi, const void* __restrict__ gf, int gate_dtype, const float* __restrict__ c,
                     const float* __restrict__ n, const float* __restrict__ m, T* __restrict__ h,
                     float* __restrict__ c_new, float* __restrict__ n_new, float* __restrict__ m_new, int Tn, int DHQK,
                     int DHHV, float eps) {
  extern __shared__ float sm[];
  float* s_q = sm;
  float* s_k = s_q + DHQK;
  float* s_n = s_k + DHQK;
  float* s_red = s_n + DHQK;
  __shared__ float s_warp[STEP_THREADS / 32];
  __shared__ float s_den;

  const int tid = threadIdx.x;
  // 1-D grid (no 65535 limit on batch x heads): the column tiles of one (batch, head) next to each other
  const int ntile = (DHHV + STEP_TV - 1) / STEP_TV;
  const int bh = blockIdx.x / ntile, tile = blockIdx.x % ntile, e0 = tile * STEP_TV;
  const int cgi = tid % STEP_CG, rg = tid / STEP_CG;
  const int e = e0 + cgi * 4;
  const float scale = rsqrtf((float)DHQK);

  float4 C[ROWS];
#pragma unroll
  for (int r = 0; r < ROWS; ++r) {
    const int d = rg + r * STEP_RG;
    C[r] = (c && d < DHQK && e < DHHV) ? *reinterpret_cast<const float4*>(c + ((size_t)bh * DHQK + d) * DHHV + e)
                                      : make_float4(0.f, 0.f, 0.f, 0.f);
  }
  for (int d = tid; d < DHQK; d += STEP_THREADS) s_n[d] = n ? n[(size_t)bh * DHQK + d] : 0.f;
  float m_run = m ? m[bh] : 0.f;
  __syncthreads();

  for (int t = 0; t < Tn; ++t) {
    const size_t tok = (size_t)bh * Tn + t;
    const float lf = logsigmoid_f(load_gate(gf, tok, gate_dtype));
    const float iv = load_gate(gi, tok, gate_dtype);
    const float m_n = fmaxf(lf + m_run, iv);
    const float fbar = expf(lf + m_run - m_n);
    const float ibar = expf(iv - m_n);
    m_run = m_n;
    float qn = 0.f;
    for (int d = tid; d < DHQK; d += STEP_THREADS) {
      const float qs = to_f32(q[tok * DHQK + d]) * scale;
      const float ik = ibar * to_f32(k[tok * DHQK + d]);
      const float nn = fmaf(fbar, s_n[d], ik);
      s_q[d] = qs; s_k[d] = ik; s_n[d] = nn;
      qn = fmaf(qs, nn, qn);
    }
    qn = warp_sum(qn);
    if ((tid & 31) == 0) s_warp[tid >> 5] = qn;
    __syncthreads();
    if (tid == 0) {
      float a = 0.f;
      for (int w = 0; w < STEP_THREADS / 32; ++w) a += s_warp[w];
      s_den = fmaxf(fabsf(a), expf(-m_n)) + eps;
    }
    float4 hv = make_float4(0.f, 0.f, 0.f, 0.f);
    if (e < DHHV) {
      const float4 vv = make_float4(to_f32(v[tok * DHHV + e]), to_f32(v[tok * DHHV + e + 1]),
                                    to_f32(v[tok * DHHV + e + 2]), to_f32(v[tok * DHHV + e + 3]));
#pragma unroll
      for (int r = 0; r < ROWS; ++r) {
        const int d = rg + r * STEP_RG;
        if (d < DHQK) {
          const float kk = s_k[d], qq = s_q[d];
          C[r].x = fmaf(fbar, C[r].x, kk * vv.x);
          C[r].y = fmaf(fbar, C[r].y, kk * vv.y);
          C[r].z = fmaf(fbar, C[r].z, kk * vv.z);
          C[r].w = fmaf(fbar, C[r].w, kk * vv.w);
          hv.x = fmaf(qq, C[r].x, hv.x); hv.y = fmaf(qq, C[r].y, hv.y);
          hv.z = fmaf(qq, C[r].z, hv.z); hv.w = fmaf(qq, C[r].w, hv.w);
        }
      }
    }
    hv.x += __shfl_xor_sync(0xffffffffu, hv.x, 16);
    hv.y += __shfl_xor_sync(0xffffffffu, hv.y, 16);
    hv.z += __shfl_xor_sync(0xffffffffu, hv.z, 16);
    hv.w += __shfl_xor_sync(0xffffffffu, hv.w, 16);
    if ((tid & 31) < 16) {
      float* dst = s_red + (tid >> 5) * STEP_TV + cgi * 4;
      dst[0] = hv.x; dst[1] = hv.y; dst[2] = hv.z; dst[3] = hv.w;
    }
    __syncthreads();
    if (tid < STEP_TV && e0 + tid < DHHV) {
      float a = 0.f;
#pragma unroll
      for (int w = 0; w < STEP_THREADS / 32; ++w) a += s_red[w * STEP_TV + tid];
      h[tok * DHHV + e0 + tid] = from_f32<T>(a / s_den);
    }
    __syncthreads();
  }
#pragma unroll
  for (int r = 0; r < ROWS; ++r) {
    const int d = rg + r * STEP_RG;
    if (d < DHQK && e < DHHV) *reinterpret_cast<float4*>(c_new + ((size_t)bh * DHQK + d) * DHHV + e) = C[r];
  }
  if (tile == 0) {
    for (int d = tid; d < DHQK; d += STEP_THREADS) n_new[(size_t)bh * DHQK + d] = s_n[d];
    if (tid == 0) m_new[bh] = m_run;
  }
}

// ---- launchers ----------------------------------------------------------------------------------------
template <typename T, typename TS>
int step_t(const void* q, const void* k, const void* v, const void* i, const void* f, int gate_dtype, const void* c,
           const void* n, const void* m, void* h, void* c_new, void* n_new, void* m_new, int B, int NH, int DHQK,
           int DHHV, float eps, cudaStream_t st) {
  PhaseScope ps(PH_STEP, st);
  const unsigned grid = (unsigned)ceil_div(DHHV, STEP_TV) * (unsigned)(B * NH);
  const size_t smem = sizeof(float) * (2 * (size_t)DHQK + (STEP_THREADS / 32) * STEP_TV);
  auto kern = step_kernel<T, TS>;
  if (smem > 48 * 1024) MLSTM_CUDA_CHECK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
  kern<<<grid, STEP_THREADS, smem, st>>>((const T*)q, (const T*)k, (const T*)v, i, f, gate_dtype,
                                         (const TS*)c, (const TS*)n, (const TS*)m, (T*)h, (TS*)c_new, (TS*)n_new,
                                         (TS*)m_new, DHQK, DHHV, eps);
  MLSTM_LAUNCH_CHECK();
  return MLSTM_OK;
}

int launch_step(const void* q, const void* k, const void* v, const void* i, const void* f, const void* c,
                const void* n, const void* m, void* h, void* c_new, void* n_new, void* m_new, int B, int NH, int DHQK,
                int DHHV, int dtype, int gate_dtype, int state_dtype, float eps, cudaStream_t st) {
#define STEP_CASE(DT, T, SDT, TS) \
  if (dtype == DT && state_dtype == SDT) return step_t<T, TS>(q, k, v, i, f, gate_dtype, c, n, m, h, c_new, n_new, m_new, B, NH, DHQK, DHHV, eps, st);
  STEP_CASE(MLSTM_F32, float, MLSTM_F32, float)
  STEP_CASE(MLSTM_BF16, __nv_bfloat16, MLSTM_F32, float)
  STEP_CASE(MLSTM_F16, __half, MLSTM_F32, float)
  STEP_CASE(MLSTM_F32, float, MLSTM_BF16, __nv_bfloat16)
  STEP_CASE(MLSTM_BF16, __nv_bfloat16, MLSTM_BF16, __nv_bfloat16)
  STEP_CASE(MLSTM_F16, __half, MLSTM_BF16, __nv_bfloat16)
#undef STEP_CASE
  return MLSTM_ERR_DTYPE;
}

template <typename T, int ROWS>
int step_seq_t(const void* q, const void* k, const void* v, const void* i, const void* f, int gate_dtype, const float* c,
               const float* n, const float* m, void* h, float* c_new, float* n_new, float* m_new, int B, int NH, int Tn,
               int DHQK, int DHHV, float eps, cudaStream_t st) {
  const unsigned grid = (unsigned)ceil_div(DHHV, STEP_TV) * (unsigned)(B * NH);
  const size_t smem = sizeof(float) * (3 * (size_t)DHQK + (STEP_THREADS / 32) * STEP_TV);
  auto kern = step_sequence_kernel<T, ROWS>;
  if (smem > 48 * 1024) MLSTM_CUDA_CHECK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
  kern<<<grid, STEP_THREADS, smem, st>>>((const T*)q, (const T*)k, (const T*)v, i, f, gate_dtype, c, n, m,
                                         (T*)h, c_new, n_new, m_new, Tn, DHQK, DHHV, eps);
  MLSTM_LAUNCH_CHECK();
  return MLSTM_OK;
}

template <typename T>
int step_seq_rows(const void* q, const void* k, const void* v, const void* i, const void* f, int gate_dtype,
                  const float* c, const float* n, const float* m, void* h, float* c_new, float* n_new, float* m_new,
                  int B, int NH, int Tn, int DHQK, int DHHV, float eps, cudaStream_t st) {
  const int rows = ceil_div(DHQK, STEP_RG);
#define SEQ_CASE(R) \
  if (rows <= R) return step_seq_t<T, R>(q, k, v, i, f, gate_dtype, c, n, m, h, c_new, n_new, m_new, B, NH, Tn, DHQK, DHHV, eps, st);
  SEQ_CASE(4) SEQ_CASE(8) SEQ_CASE(16) SEQ_CASE(32)
#undef SEQ_CASE
  return MLSTM_ERR_SHAPE;
}

int launch_step_sequence(const void* q, const void* k, const void* v, const void* i, const void* f, const float* c,
                         const float* n, const float* m, void* h, float* c_new, float* n_new, float* m_new, int B,
                         int NH, int T, int DHQK, int DHHV, int dtype, int gate_dtype, float eps, cudaStream_t st) {
  switch (dtype) {
    case MLSTM_F32: return step_seq_rows<float>(q, k, v, i, f, gate_dtype, c, n, m, h, c_new, n_new, m_new, B, NH, T, DHQK, DHHV, eps, st);
    case MLSTM_BF16: return step_seq_rows<__nv_bfloat16>(q, k, v, i, f, gate_dtype, c, n, m, h, c_new, n_new, m_new, B, NH, T, DHQK, DHHV, eps, st);
    case MLSTM_F16: return step_seq_rows<__half>(q, k, v, i, f, gate_dtype, c, n, m, h, c_new, n_new, m_new, B, NH, T, DHQK, DHHV, eps, st);
  }
  return MLSTM_ERR_DTYPE;
}

}  // namespace mlstm
