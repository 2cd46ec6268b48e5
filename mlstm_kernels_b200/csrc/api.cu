// extern "C" entry points of libmlstm_b200.so: argument validation, workspace carving, dispatch.
#include <algorithm>
#include <atomic>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <mutex>
#include <vector>

#include <nvtx3/nvToolsExt.h>

#include "common.cuh"
#include "launch.cuh"

namespace mlstm {

static thread_local char g_last_cuda_error[512] = "";

void set_last_cuda_error(cudaError_t e, const char* where) {
  snprintf(g_last_cuda_error, sizeof(g_last_cuda_error), "%s: %s (%s)", cudaGetErrorName(e), cudaGetErrorString(e),
           where);
}

// ---- launch counter and phase profiler ----------------------------------------------------------
static std::atomic<long long> g_launches{0};
void note_launch() { g_launches.fetch_add(1, std::memory_order_relaxed); }

struct PhaseRec { int phase; cudaEvent_t a, b; };
static std::mutex g_prof_mu;
static bool g_prof_on = false;
static std::vector<PhaseRec> g_prof_recs;
static const size_t kMaxPhaseRecs = 1 << 16;

// NVTX ranges around the phases (mlstm_b200_nvtx_enable): host-side markers for a timeline profiler, named like the
// phases of mlstm_b200_profile_phase_name.  Off by default; the header-only NVTX loads the tools library on first use.
static std::atomic<int> g_nvtx_on{0};
static const char* const kPhaseNames[PH_COUNT] = {"gates", "recurrent_fw", "parallel_fw", "recurrent_bw",
                                                   "parallel_bw", "gate_grads", "step"};

PhaseScope::PhaseScope(int phase, cudaStream_t s) : slot(-1), st(s), nvtx(false) {
  if (g_nvtx_on.load(std::memory_order_relaxed) != 0 && phase >= 0 && phase < PH_COUNT) {
    nvtxRangePushA(kPhaseNames[phase]);
    nvtx = true;
  }
  if (!g_prof_on) return;
  std::lock_guard<std::mutex> lk(g_prof_mu);
  if (g_prof_recs.size() >= kMaxPhaseRecs) return;
  PhaseRec r{phase, nullptr, nullptr};
  if (cudaEventCreate(&r.a) != cudaSuccess || cudaEventCreate(&r.b) != cudaSuccess) return;
  cudaEventRecord(r.a, st);
  g_prof_recs.push_back(r);
  slot = (int)g_prof_recs.size() - 1;
}
PhaseScope::~PhaseScope() {
  if (nvtx) nvtxRangePop();
  if (slot < 0) return;
  std::lock_guard<std::mutex> lk(g_prof_mu);
  if (slot < (int)g_prof_recs.size()) cudaEventRecord(g_prof_recs[slot].b, st);
}

static bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

// ---- the (batch, head) units as two chains of launches on two streams ---------------------------------
// Each recurrence CTA walks a whole sequence, so a launch whose CTA count is not a multiple of the SM count ends with
// a partly filled wave, and the intra-chunk kernel behind it waits for that wave.  The units are independent: the
// first half runs on the caller's stream and the second half on a stream of the library, forked and joined with
// events (the pattern stream capture allows), and the block scheduler fills the idle SMs of one chain's last wave
// with the other chain's CTAs.  No kernel waits for another one: the order is the streams' and events' only.
struct SideStream { cudaStream_t st = nullptr; cudaEvent_t fork = nullptr, join = nullptr; };
static std::mutex g_side_mu;          // held while a split call enqueues: one stream and one event pair per device
static SideStream g_side[64];
static std::atomic<int> g_split_on{1};

static SideStream* side_stream_for_current_device() {
  int dev = -1;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return nullptr;
  SideStream& s = g_side[dev];
  if (s.st == nullptr) {
    cudaStream_t st = nullptr;
    cudaEvent_t a = nullptr, b = nullptr;
    // default priority: giving this stream a higher one (so that the second half's recurrence CTAs are placed before
    // the first half's intra-chunk CTAs) measured slower
    if (cudaStreamCreateWithFlags(&st, cudaStreamNonBlocking) != cudaSuccess ||
        cudaEventCreateWithFlags(&a, cudaEventDisableTiming) != cudaSuccess ||
        cudaEventCreateWithFlags(&b, cudaEventDisableTiming) != cudaSuccess) {
      (void)cudaGetLastError();
      if (st) cudaStreamDestroy(st);
      if (a) cudaEventDestroy(a);
      if (b) cudaEventDestroy(b);
      return nullptr;
    }
    s.st = st; s.fork = a; s.join = b;
  }
  return &s;
}

// worth it only when the recurrence needs more than one wave of CTAs and the last one is far from full (and never
// while phases are being timed)
static bool want_unit_split(const ChunkwiseDims& d, bool allow) {
  if (!allow || g_split_on.load(std::memory_order_relaxed) == 0 || g_prof_on || d.B * d.NH < 2) return false;
  const long ctas = sm100_recurrence_ctas(d), sms = sm100_sm_count();
  const long waves = (ctas + sms - 1) / sms;
  return waves > 1 && ctas * 100 < waves * sms * 95;   // the last wave leaves more than 5 % of the SM time idle
}

// Fork on construction (when the split is wanted and the second stream exists), join on join() or, if an error path
// leaves the scope early, in the destructor - a stream that is being captured must never be left forked.
class UnitChains {
 public:
  UnitChains(const ChunkwiseDims& d, cudaStream_t st, bool allow) : st_(st), lk_(g_side_mu, std::defer_lock) {
    const int units = d.B * d.NH;
    first_ = UnitRange{0, units};
    if (!want_unit_split(d, allow)) return;
    lk_.lock();
    SideStream* s = side_stream_for_current_device();
    if (s == nullptr) { lk_.unlock(); return; }
    if (cudaEventRecord(s->fork, st_) != cudaSuccess || cudaStreamWaitEvent(s->st, s->fork, 0) != cudaSuccess) {
      set_last_cuda_error(cudaGetLastError(), "fork of the second launch chain");
      rc_ = MLSTM_ERR_CUDA;
      lk_.unlock();
      return;
    }
    side_ = s;
    first_ = UnitRange{0, (units + 1) / 2};
    second_ = UnitRange{first_.count, -1};
  }
  ~UnitChains() { (void)join(); }
  UnitChains(const UnitChains&) = delete;
  UnitChains& operator=(const UnitChains&) = delete;
  int status() const { return rc_; }
  bool split() const { return side_ != nullptr; }
  cudaStream_t second_stream() const { return side_->st; }
  UnitRange first() const { return first_; }
  UnitRange second() const { return second_; }
  int join() {
    if (side_ == nullptr) return MLSTM_OK;
    SideStream* s = side_;
    side_ = nullptr;
    const bool ok = cudaEventRecord(s->join, s->st) == cudaSuccess && cudaStreamWaitEvent(st_, s->join, 0) == cudaSuccess;
    if (!ok) set_last_cuda_error(cudaGetLastError(), "join of the second launch chain");
    lk_.unlock();
    return ok ? MLSTM_OK : MLSTM_ERR_CUDA;
  }

 private:
  cudaStream_t st_;
  std::unique_lock<std::mutex> lk_;
  SideStream* side_ = nullptr;
  UnitRange first_, second_;
  int rc_ = MLSTM_OK;
};

// S need not be a multiple of L where the tcgen05 kernels run (they mask a ragged last chunk); resolve_impl refuses
// that case for the portable kernels.
static int check_dims(int B, int NH, int S, int DHQK, int DHHV, int L) {
  if (B <= 0 || NH <= 0 || S <= 0 || DHQK <= 0 || DHHV <= 0 || L <= 0) return MLSTM_ERR_SHAPE;
  if (!is_pow2(L) || L < 16 || L > 1024) return MLSTM_ERR_SHAPE;
  // Sizes the launches cannot express are refused here instead of failing at launch or overflowing an index:
  // the grids carry (tiles x chunks x batch x heads) in one dimension, and the tcgen05 kernels address token and
  // state rows with 32-bit coordinates.
  const uint64_t lim = 0x7fffffffull;
  const uint64_t bnh = (uint64_t)B * NH, nc = ((uint64_t)S + L - 1) / L;
  const uint64_t tiles = (uint64_t)std::max(ceil_div(DHQK, 64), ceil_div(DHHV, 64));
  if (bnh * nc * tiles >= lim || bnh * S >= lim) return MLSTM_ERR_SHAPE;
  return MLSTM_OK;
}

static int resolve_impl(int impl, int B, int NH, int S, int DHQK, int DHHV, int L, int dtype, bool* use_sm100) {
  const bool ok = sm100_supported(S, DHQK, DHHV, L, dtype);
  if (impl != MLSTM_IMPL_AUTO && impl != MLSTM_IMPL_SIMT && impl != MLSTM_IMPL_TCGEN05) return MLSTM_ERR_UNSUPPORTED;
  *use_sm100 = ok && impl != MLSTM_IMPL_SIMT;
  if (impl == MLSTM_IMPL_TCGEN05 && !ok) return MLSTM_ERR_UNSUPPORTED;
  if (*use_sm100 && !sm100_sizes_ok(B, NH, S, DHQK, DHHV)) return MLSTM_ERR_SHAPE;
  if (!*use_sm100 && S % L != 0) return MLSTM_ERR_SHAPE;   // the portable kernels need whole chunks
  return MLSTM_OK;
}

// carve f32 arrays out of the workspace, each start 256-byte aligned
struct Carver {
  char* base; size_t off = 0;
  explicit Carver(void* p) : base(static_cast<char*>(p)) {}
  template <typename T> T* take(size_t count) {
    off = align_up(off, 256);
    T* p = base ? reinterpret_cast<T*>(base + off) : nullptr;
    off += count * sizeof(T);
    return p;
  }
};

struct FwLayout { GateBuffers gb; size_t bytes; };
// per-token arrays have SP = NC * L slots per (batch, head)
static FwLayout carve_fw(void* ws, int BNH, int SP, int NC) {
  Carver c(ws);
  FwLayout l{};
  const size_t tok = (size_t)BNH * SP;
  l.gb.vecB = c.take<float>(tok);
  l.gb.iota = c.take<float>(tok);
  l.gb.abar = c.take<float>(tok);
  l.gb.bbar = c.take<float>(tok);
  l.gb.m_tok = c.take<float>(tok);
  l.gb.gbar = c.take<float>((size_t)BNH * NC);
  l.gb.scratch = c.take<float>((size_t)BNH * NC * 2);
  l.gb.inv_den = nullptr;
  l.bytes = align_up(c.off, 256);
  return l;
}

struct SumLayout { GateBuffers gb; float* m_states; size_t bytes; };
static SumLayout carve_summary(void* ws, int BNH, int SP, int NC) {
  Carver c(ws);
  SumLayout l{};
  const size_t tok = (size_t)BNH * SP;
  l.gb.vecB = c.take<float>(tok);
  l.gb.iota = c.take<float>(tok);
  l.gb.m_tok = c.take<float>(tok);
  l.gb.abar = c.take<float>(tok);
  l.gb.bbar = c.take<float>(tok);
  l.gb.gbar = c.take<float>((size_t)BNH * NC);
  l.gb.scratch = c.take<float>((size_t)BNH * NC * 2);
  l.gb.inv_den = nullptr;
  l.m_states = c.take<float>((size_t)BNH * (NC + 1));
  l.bytes = align_up(c.off, 256);
  return l;
}

// every kAnchorEvery-th chunk boundary carries an exact value of the forget-gate gradient's running sum
constexpr int kAnchorEvery = 4;
static int anchor_count(int NC) { return (NC + kAnchorEvery - 1) / kAnchorEvery + 1; }

struct BwLayout { GateBuffers gb; float* m_states; float* acc; float* kdk; float* anchors; void* dc_states; size_t bytes; };
static BwLayout carve_bw(void* ws, int BNH, int SP, int NC, int DHQK, int DHHV, size_t state_elem) {
  Carver c(ws);
  BwLayout l{};
  const size_t tok = (size_t)BNH * SP;
  l.gb.vecB = c.take<float>(tok);
  l.gb.iota = c.take<float>(tok);
  l.gb.m_tok = c.take<float>(tok);
  l.gb.abar = c.take<float>(tok);
  l.gb.bbar = c.take<float>(tok);
  l.gb.inv_den = c.take<float>(tok);
  l.gb.gbar = c.take<float>((size_t)BNH * NC);
  l.gb.scratch = c.take<float>((size_t)BNH * NC * 2);
  l.m_states = c.take<float>((size_t)BNH * (NC + 1));
  const size_t parts = (size_t)(DHQK + 127) / 128;  // one partial row sum per 128-wide tile of DHQK
  l.acc = c.take<float>(tok * parts);
  l.kdk = c.take<float>(tok * parts);
  l.anchors = c.take<float>((size_t)BNH * anchor_count(NC));
  l.dc_states = c.take<char>((size_t)BNH * (NC + 1) * DHQK * DHHV * state_elem);
  l.bytes = align_up(c.off, 256);
  return l;
}

}  // namespace mlstm

using namespace mlstm;

extern "C" {

int mlstm_b200_version(void) { return 100; }

const char* mlstm_b200_error_string(int code) {
  switch (code) {
    case MLSTM_OK: return "ok";
    case MLSTM_ERR_SHAPE: return "unsupported or inconsistent sizes";
    case MLSTM_ERR_DTYPE: return "unsupported element type";
    case MLSTM_ERR_NULL: return "a required pointer is NULL";
    case MLSTM_ERR_ALIGN: return "a pointer is not 16-byte aligned";
    case MLSTM_ERR_WORKSPACE: return "workspace too small";
    case MLSTM_ERR_CUDA: return "a CUDA call failed";
    case MLSTM_ERR_UNSUPPORTED: return "requested implementation cannot run this case";
  }
  return "unknown error code";
}

const char* mlstm_b200_last_cuda_error(void) { return g_last_cuda_error; }

long long mlstm_b200_launch_count(void) { return g_launches.load(); }

int mlstm_b200_device_status(int reset) {
  int status = 0;
  const int rc = sm100_device_status(reset, &status);
  return rc != MLSTM_OK ? rc : status;
}

int mlstm_b200_selftest_wait_expiry(unsigned int limit_polls, int code, void* stream) {
  return sm100_wait_expiry_selftest(limit_polls, code, static_cast<cudaStream_t>(stream));
}

int mlstm_b200_profile_enable(int on) {
  std::lock_guard<std::mutex> lk(g_prof_mu);
  for (auto& r : g_prof_recs) { cudaEventDestroy(r.a); cudaEventDestroy(r.b); }
  g_prof_recs.clear();
  g_prof_on = on != 0;
  return MLSTM_OK;
}

int mlstm_b200_profile_phases(void) { return PH_COUNT; }

const char* mlstm_b200_profile_phase_name(int phase) {
  return (phase >= 0 && phase < PH_COUNT) ? kPhaseNames[phase] : "?";
}

int mlstm_b200_nvtx_enable(int on) { return g_nvtx_on.exchange(on != 0 ? 1 : 0); }

int mlstm_b200_profile_read(float* total_ms, int* count) {
  std::lock_guard<std::mutex> lk(g_prof_mu);
  for (int p = 0; p < PH_COUNT; ++p) { total_ms[p] = 0.f; count[p] = 0; }
  for (auto& r : g_prof_recs) {
    MLSTM_CUDA_CHECK(cudaEventSynchronize(r.b));
    float ms = 0.f;
    MLSTM_CUDA_CHECK(cudaEventElapsedTime(&ms, r.a, r.b));
    total_ms[r.phase] += ms;
    count[r.phase] += 1;
  }
  for (auto& r : g_prof_recs) { cudaEventDestroy(r.a); cudaEventDestroy(r.b); }
  g_prof_recs.clear();
  return MLSTM_OK;
}

int mlstm_b200_chunkwise_has_tcgen05(int S, int DHQK, int DHHV, int L, int dtype) {
  return sm100_supported(S, DHQK, DHHV, L, dtype) ? 1 : 0;
}

int mlstm_b200_chunkwise_state_dtype(int S, int DHQK, int DHHV, int L, int dtype, int impl) {
  bool use_sm100 = false;
  if (resolve_impl(impl, 1, 1, S, DHQK, DHHV, L, dtype, &use_sm100) != MLSTM_OK) return MLSTM_F32;
  return use_sm100 ? dtype : MLSTM_F32;   // tcgen05 path: 16-bit states of the input type
}

size_t mlstm_b200_chunkwise_workspace_bytes(int B, int NH, int S, int DHQK, int DHHV, int L, int dtype, int variant,
                                            int impl, int backward) {
  (void)variant;
  if (check_dims(B, NH, S, DHQK, DHHV, L) != MLSTM_OK) return 0;
  bool use_sm100 = false;
  if (resolve_impl(impl, B, NH, S, DHQK, DHHV, L, dtype, &use_sm100) != MLSTM_OK) return 0;
  const int NC = (S + L - 1) / L, SP = NC * L;
  if (backward == 2) return carve_summary(nullptr, B * NH, SP, NC).bytes;
  if (!backward) return carve_fw(nullptr, B * NH, SP, NC).bytes;
  return carve_bw(nullptr, B * NH, SP, NC, DHQK, DHHV, dtype_size(use_sm100 ? dtype : MLSTM_F32)).bytes;
}

int mlstm_b200_set_unit_split(int on) { return g_split_on.exchange(on != 0 ? 1 : 0); }

int mlstm_b200_chunkwise_fw(const void* q, const void* k, const void* v, const void* i, const void* f,
                            const float* c_initial, const float* n_initial, const float* m_initial, void* h,
                            float* n_out, float* m_out, void* c_states, float* n_states, float* m_states,
                            float* c_last, float* n_last, float* m_last, void* workspace, size_t workspace_bytes,
                            int B, int NH, int S, int DHQK, int DHHV, int L, int dtype, int gate_dtype, int variant,
                            int impl, float eps, void* stream) {
  return chunkwise_fw_body(q, k, v, i, f, c_initial, n_initial, m_initial, h, n_out, m_out, c_states, n_states, m_states,
                           c_last, n_last, m_last, workspace, workspace_bytes, B, NH, S, DHQK, DHHV, L, dtype,
                           gate_dtype, variant, impl, eps, stream, true);
}

}  // extern "C"

namespace mlstm {
int chunkwise_fw_body(const void* q, const void* k, const void* v, const void* i, const void* f,
                      const float* c_initial, const float* n_initial, const float* m_initial, void* h,
                      float* n_out, float* m_out, void* c_states, float* n_states, float* m_states,
                      float* c_last, float* n_last, float* m_last, void* workspace, size_t workspace_bytes,
                      int B, int NH, int S, int DHQK, int DHHV, int L, int dtype, int gate_dtype, int variant,
                      int impl, float eps, void* stream, bool allow_split) {
  int rc = check_dims(B, NH, S, DHQK, DHHV, L);
  if (rc != MLSTM_OK) return rc;
  if (dtype != MLSTM_F32 && dtype != MLSTM_BF16 && dtype != MLSTM_F16) return MLSTM_ERR_DTYPE;
  if (gate_dtype != MLSTM_F32 && gate_dtype != MLSTM_BF16 && gate_dtype != MLSTM_F16) return MLSTM_ERR_DTYPE;
  if (variant < MLSTM_EXP || variant > MLSTM_SIG_NONORM) return MLSTM_ERR_UNSUPPORTED;
  if (!q || !k || !v || !i || !f || !h || !n_out || !m_out || !c_states || !n_states || !m_states || !workspace)
    return MLSTM_ERR_NULL;
  const void* ptrs[] = {q, k, v, i, f, c_initial, n_initial, m_initial, h, n_out, m_out, c_states, n_states, m_states,
                        c_last, n_last, m_last, workspace};
  for (const void* p : ptrs) if (p && !aligned16(p)) return MLSTM_ERR_ALIGN;
  bool use_sm100 = false;
  if ((rc = resolve_impl(impl, B, NH, S, DHQK, DHHV, L, dtype, &use_sm100)) != MLSTM_OK) return rc;

  const ChunkwiseDims d = make_dims(B, NH, S, DHQK, DHHV, L, variant, eps, dtype);
  FwLayout lay = carve_fw(workspace, B * NH, d.SP, d.NC);
  if (workspace_bytes < lay.bytes) return MLSTM_ERR_WORKSPACE;
  cudaStream_t st = static_cast<cudaStream_t>(stream);

  if ((rc = launch_gates(gate_dtype, i, f, variant == MLSTM_EXP ? m_initial : nullptr, nullptr, m_out, lay.gb, m_states, d, st)) != MLSTM_OK) return rc;
  if (use_sm100) {
    UnitChains ch(d, st, allow_split);
    if ((rc = ch.status()) != MLSTM_OK) return rc;
    if ((rc = sm100_recurrent_fw(k, v, lay.gb, c_initial, n_initial, c_states, n_states, c_last, n_last, d, st, ch.first())) != MLSTM_OK) return rc;
    if (ch.split() && (rc = sm100_recurrent_fw(k, v, lay.gb, c_initial, n_initial, c_states, n_states, c_last, n_last, d, ch.second_stream(), ch.second())) != MLSTM_OK) return rc;
    if ((rc = sm100_parallel_fw(q, k, v, lay.gb, c_states, n_states, h, n_out, d, st, ch.first())) != MLSTM_OK) return rc;
    if (ch.split() && (rc = sm100_parallel_fw(q, k, v, lay.gb, c_states, n_states, h, n_out, d, ch.second_stream(), ch.second())) != MLSTM_OK) return rc;
    if ((rc = ch.join()) != MLSTM_OK) return rc;
  } else {
    if ((rc = simt_recurrent_fw(dtype, MLSTM_F32, k, v, lay.gb, c_initial, n_initial, c_states, n_states, c_last, n_last, d, st)) != MLSTM_OK) return rc;
    if ((rc = simt_parallel_fw(dtype, MLSTM_F32, q, k, v, lay.gb, c_states, n_states, h, n_out, d, st)) != MLSTM_OK) return rc;
  }
  if (m_last) {
    MLSTM_CUDA_CHECK(cudaMemcpy2DAsync(m_last, sizeof(float), m_states + d.NC, sizeof(float) * (d.NC + 1),
                                       sizeof(float), (size_t)B * NH, cudaMemcpyDeviceToDevice, st));
  }
  return MLSTM_OK;
}
}  // namespace mlstm

// Backward body.  With `fw_workspace` (the scratch buffer the forward call of the same problem left behind, still
// intact) and `m_out` the gate pre-pass is not run again: its vectors are read from that buffer.
static int bw_impl(const void* q, const void* k, const void* v, const void* i, const void* f,
                   const float* m_initial, const void* c_states, const float* n_out, const void* dh,
                   const float* dc_last, void* dq, void* dk, void* dv, float* di, float* df,
                   float* dc_initial, void* workspace, size_t workspace_bytes, int B, int NH, int S, int DHQK,
                   int DHHV, int L, int dtype, int gate_dtype, int variant, int impl, float eps, void* stream,
                   const void* fw_workspace, size_t fw_workspace_bytes, const float* m_out,
                   void* recompute_into = nullptr, const float* recompute_c_initial = nullptr) {
  int rc = check_dims(B, NH, S, DHQK, DHHV, L);
  if (rc != MLSTM_OK) return rc;
  if (dtype != MLSTM_F32 && dtype != MLSTM_BF16 && dtype != MLSTM_F16) return MLSTM_ERR_DTYPE;
  if (gate_dtype != MLSTM_F32 && gate_dtype != MLSTM_BF16 && gate_dtype != MLSTM_F16) return MLSTM_ERR_DTYPE;
  if (variant < MLSTM_EXP || variant > MLSTM_SIG_NONORM) return MLSTM_ERR_UNSUPPORTED;
  if (!q || !k || !v || !i || !f || !c_states || !dh || !dq || !dk || !dv || !di || !df || !workspace)
    return MLSTM_ERR_NULL;
  if (variant != MLSTM_SIG_NONORM && !n_out) return MLSTM_ERR_NULL;
  const void* ptrs[] = {q, k, v, i, f, m_initial, c_states, n_out, dh, dc_last, dq, dk, dv, di, df, dc_initial, workspace,
                        recompute_c_initial};
  for (const void* p : ptrs) if (p && !aligned16(p)) return MLSTM_ERR_ALIGN;
  // recompute_into (== c_states, writable): the per-chunk states are not there yet; the forward's recurrence is run
  // again in front of each chain of backward launches.  Needs the forward's gate vectors (fw_workspace).
  if (recompute_into != nullptr && fw_workspace == nullptr) return MLSTM_ERR_NULL;
  bool use_sm100 = false;
  if ((rc = resolve_impl(impl, B, NH, S, DHQK, DHHV, L, dtype, &use_sm100)) != MLSTM_OK) return rc;

  const ChunkwiseDims d = make_dims(B, NH, S, DHQK, DHHV, L, variant, eps, dtype);
  const int sdt = use_sm100 ? dtype : MLSTM_F32;
  BwLayout lay = carve_bw(workspace, B * NH, d.SP, d.NC, DHQK, DHHV, dtype_size(sdt));
  if (workspace_bytes < lay.bytes) return MLSTM_ERR_WORKSPACE;
  cudaStream_t st = static_cast<cudaStream_t>(stream);

  if (fw_workspace != nullptr) {
    if (!aligned16(fw_workspace)) return MLSTM_ERR_ALIGN;
    FwLayout fl = carve_fw(const_cast<void*>(fw_workspace), B * NH, d.SP, d.NC);
    if (fw_workspace_bytes < fl.bytes) return MLSTM_ERR_WORKSPACE;
    float* inv_den = lay.gb.inv_den;
    lay.gb = fl.gb;
    lay.gb.inv_den = inv_den;
    if ((rc = launch_inv_den(n_out, inv_den, d, st)) != MLSTM_OK) return rc;
  } else {
    if ((rc = launch_gates(gate_dtype, i, f, variant == MLSTM_EXP ? m_initial : nullptr, n_out, nullptr, lay.gb, lay.m_states, d, st)) != MLSTM_OK) return rc;
  }
  if (use_sm100) {
    {
      UnitChains ch(d, st, true);
      if ((rc = ch.status()) != MLSTM_OK) return rc;
      if (recompute_into) {
        if ((rc = sm100_recurrent_fw(k, v, lay.gb, recompute_c_initial, nullptr, recompute_into, nullptr, nullptr, nullptr, d, st, ch.first())) != MLSTM_OK) return rc;
        if (ch.split() && (rc = sm100_recurrent_fw(k, v, lay.gb, recompute_c_initial, nullptr, recompute_into, nullptr, nullptr, nullptr, d, ch.second_stream(), ch.second())) != MLSTM_OK) return rc;
      }
      if ((rc = sm100_recurrent_bw(q, dh, lay.gb, dc_last, lay.dc_states, dc_initial, d, st, ch.first())) != MLSTM_OK) return rc;
      if (ch.split() && (rc = sm100_recurrent_bw(q, dh, lay.gb, dc_last, lay.dc_states, dc_initial, d, ch.second_stream(), ch.second())) != MLSTM_OK) return rc;
      if ((rc = sm100_parallel_bw(q, k, v, dh, lay.gb, c_states, lay.dc_states, dq, dk, dv, lay.acc, lay.kdk, d, st, ch.first())) != MLSTM_OK) return rc;
      if (ch.split() && (rc = sm100_parallel_bw(q, k, v, dh, lay.gb, c_states, lay.dc_states, dq, dk, dv, lay.acc, lay.kdk, d, ch.second_stream(), ch.second())) != MLSTM_OK) return rc;
      if ((rc = ch.join()) != MLSTM_OK) return rc;
    }
    {
      PhaseScope ps(PH_GATE_GRADS, st);
      const int n_anchors = anchor_count(d.NC);
      // (sequences of up to kAnchorEvery chunks have no interior anchor: nothing to compute)
      if (n_anchors > 2 &&
          (rc = launch_state_dot(c_states, lay.dc_states, lay.anchors, kAnchorEvery, n_anchors, d, st)) != MLSTM_OK) return rc;
      if ((rc = launch_gate_grad_scan(gate_dtype, i, f, lay.acc, lay.kdk, (DHQK + 127) / 128, di, df, d, st, lay.anchors,
                                      n_anchors, kAnchorEvery * L)) != MLSTM_OK) return rc;
    }
  } else {
    if (recompute_into &&
        (rc = simt_recurrent_fw(dtype, MLSTM_F32, k, v, lay.gb, recompute_c_initial, nullptr, recompute_into, nullptr, nullptr, nullptr, d, st)) != MLSTM_OK) return rc;
    if ((rc = simt_recurrent_bw(dtype, sdt, q, dh, lay.gb, dc_last, lay.dc_states, dc_initial, d, st)) != MLSTM_OK) return rc;
    if ((rc = simt_parallel_bw(dtype, sdt, q, k, v, dh, lay.gb, c_states, lay.dc_states, dq, dk, dv, d, st)) != MLSTM_OK) return rc;
    if ((rc = launch_gate_grads(dtype, gate_dtype, q, k, dq, dk, i, f, lay.acc, lay.kdk, di, df, d, st)) != MLSTM_OK) return rc;
  }
  return MLSTM_OK;
}

extern "C" {

int mlstm_b200_chunkwise_bw(const void* q, const void* k, const void* v, const void* i, const void* f,
                            const float* m_initial, const void* c_states, const float* n_out, const void* dh,
                            const float* dc_last, void* dq, void* dk, void* dv, float* di, float* df,
                            float* dc_initial, void* workspace, size_t workspace_bytes, int B, int NH, int S, int DHQK,
                            int DHHV, int L, int dtype, int gate_dtype, int variant, int impl, float eps, void* stream) {
  return bw_impl(q, k, v, i, f, m_initial, c_states, n_out, dh, dc_last, dq, dk, dv, di, df, dc_initial, workspace,
                 workspace_bytes, B, NH, S, DHQK, DHHV, L, dtype, gate_dtype, variant, impl, eps, stream, nullptr, 0,
                 nullptr);
}

int mlstm_b200_chunkwise_bw_cached(const void* q, const void* k, const void* v, const void* i, const void* f,
                                   const float* m_initial, const void* c_states, const float* n_out,
                                   const float* m_out, const void* fw_workspace, size_t fw_workspace_bytes,
                                   const void* dh, const float* dc_last, void* dq, void* dk, void* dv, float* di,
                                   float* df, float* dc_initial, void* workspace, size_t workspace_bytes, int B,
                                   int NH, int S, int DHQK, int DHHV, int L, int dtype, int gate_dtype, int variant,
                                   int impl, float eps, void* stream) {
  if (!fw_workspace) return MLSTM_ERR_NULL;
  return bw_impl(q, k, v, i, f, m_initial, c_states, n_out, dh, dc_last, dq, dk, dv, di, df, dc_initial, workspace,
                 workspace_bytes, B, NH, S, DHQK, DHHV, L, dtype, gate_dtype, variant, impl, eps, stream, fw_workspace,
                 fw_workspace_bytes, m_out);
}

int mlstm_b200_chunkwise_bw_recompute(const void* q, const void* k, const void* v, const void* i, const void* f,
                                      const float* m_initial, const float* c_initial, void* c_states_scratch,
                                      const float* n_out, const float* m_out, const void* fw_workspace,
                                      size_t fw_workspace_bytes, const void* dh, const float* dc_last, void* dq,
                                      void* dk, void* dv, float* di, float* df, float* dc_initial, void* workspace,
                                      size_t workspace_bytes, int B, int NH, int S, int DHQK, int DHHV, int L,
                                      int dtype, int gate_dtype, int variant, int impl, float eps, void* stream) {
  if (!fw_workspace || !c_states_scratch) return MLSTM_ERR_NULL;
  return bw_impl(q, k, v, i, f, m_initial, c_states_scratch, n_out, dh, dc_last, dq, dk, dv, di, df, dc_initial,
                 workspace, workspace_bytes, B, NH, S, DHQK, DHHV, L, dtype, gate_dtype, variant, impl, eps, stream,
                 fw_workspace, fw_workspace_bytes, m_out, c_states_scratch, c_initial);
}

int mlstm_b200_chunkwise_states(const void* k, const void* v, const void* i, const void* f, const float* c_initial,
                                const float* m_initial, void* c_states, const void* fw_workspace,
                                size_t fw_workspace_bytes, void* workspace, size_t workspace_bytes, int B, int NH,
                                int S, int DHQK, int DHHV, int L, int dtype, int gate_dtype, int variant, int impl,
                                void* stream) {
  int rc = check_dims(B, NH, S, DHQK, DHHV, L);
  if (rc != MLSTM_OK) return rc;
  if (dtype != MLSTM_F32 && dtype != MLSTM_BF16 && dtype != MLSTM_F16) return MLSTM_ERR_DTYPE;
  if (gate_dtype != MLSTM_F32 && gate_dtype != MLSTM_BF16 && gate_dtype != MLSTM_F16) return MLSTM_ERR_DTYPE;
  if (variant < MLSTM_EXP || variant > MLSTM_SIG_NONORM) return MLSTM_ERR_UNSUPPORTED;
  if (!k || !v || !i || !f || !c_states) return MLSTM_ERR_NULL;
  if (!fw_workspace && !workspace) return MLSTM_ERR_NULL;
  const void* ptrs[] = {k, v, i, f, c_initial, m_initial, c_states, fw_workspace, workspace};
  for (const void* p : ptrs) if (p && !aligned16(p)) return MLSTM_ERR_ALIGN;
  bool use_sm100 = false;
  if ((rc = resolve_impl(impl, B, NH, S, DHQK, DHHV, L, dtype, &use_sm100)) != MLSTM_OK) return rc;
  const ChunkwiseDims d = make_dims(B, NH, S, DHQK, DHHV, L, variant, 1e-6f, dtype);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  GateBuffers gb;
  if (fw_workspace != nullptr) {   // the forward's gate vectors are still there: only abar and gbar are read
    FwLayout fl = carve_fw(const_cast<void*>(fw_workspace), B * NH, d.SP, d.NC);
    if (fw_workspace_bytes < fl.bytes) return MLSTM_ERR_WORKSPACE;
    gb = fl.gb;
  } else {
    SumLayout lay = carve_summary(workspace, B * NH, d.SP, d.NC);
    if (workspace_bytes < lay.bytes) return MLSTM_ERR_WORKSPACE;
    gb = lay.gb;
    if ((rc = launch_gates(gate_dtype, i, f, variant == MLSTM_EXP ? m_initial : nullptr, nullptr, nullptr, gb, lay.m_states, d, st)) != MLSTM_OK) return rc;
  }
  if (use_sm100) return sm100_recurrent_fw(k, v, gb, c_initial, nullptr, c_states, nullptr, nullptr, nullptr, d, st);
  return simt_recurrent_fw(dtype, MLSTM_F32, k, v, gb, c_initial, nullptr, c_states, nullptr, nullptr, nullptr, d, st);
}

int mlstm_b200_chunkwise_dc_summary(const void* q, const void* dh, const float* n_out, const void* fw_workspace,
                                    size_t fw_workspace_bytes, float* dc_initial, void* workspace,
                                    size_t workspace_bytes, int B, int NH, int S, int DHQK, int DHHV, int L, int dtype,
                                    int variant, int impl, float eps, void* stream) {
  int rc = check_dims(B, NH, S, DHQK, DHHV, L);
  if (rc != MLSTM_OK) return rc;
  if (dtype != MLSTM_F32 && dtype != MLSTM_BF16 && dtype != MLSTM_F16) return MLSTM_ERR_DTYPE;
  if (variant < MLSTM_EXP || variant > MLSTM_SIG_NONORM) return MLSTM_ERR_UNSUPPORTED;
  if (!q || !dh || !fw_workspace || !dc_initial || !workspace) return MLSTM_ERR_NULL;
  if (variant != MLSTM_SIG_NONORM && !n_out) return MLSTM_ERR_NULL;
  const void* ptrs[] = {q, dh, n_out, fw_workspace, dc_initial, workspace};
  for (const void* p : ptrs) if (p && !aligned16(p)) return MLSTM_ERR_ALIGN;
  bool use_sm100 = false;
  if ((rc = resolve_impl(impl, B, NH, S, DHQK, DHHV, L, dtype, &use_sm100)) != MLSTM_OK) return rc;
  const ChunkwiseDims d = make_dims(B, NH, S, DHQK, DHHV, L, variant, eps, dtype);
  FwLayout fl = carve_fw(const_cast<void*>(fw_workspace), B * NH, d.SP, d.NC);
  if (fw_workspace_bytes < fl.bytes) return MLSTM_ERR_WORKSPACE;
  const size_t need = align_up((size_t)B * NH * d.SP * sizeof(float), 256);
  if (workspace_bytes < need) return MLSTM_ERR_WORKSPACE;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  GateBuffers gb = fl.gb;
  gb.inv_den = static_cast<float*>(workspace);
  if ((rc = launch_inv_den(n_out, gb.inv_den, d, st)) != MLSTM_OK) return rc;
  if (use_sm100) return sm100_recurrent_bw(q, dh, gb, nullptr, nullptr, dc_initial, d, st);
  return simt_recurrent_bw(dtype, MLSTM_F32, q, dh, gb, nullptr, nullptr, dc_initial, d, st);
}

int mlstm_b200_chunkwise_summary(const void* k, const void* v, const void* i, const void* f, float* c_last,
                                 float* n_last, float* m_last, float* g_total, void* workspace,
                                 size_t workspace_bytes, int B, int NH, int S, int DHQK, int DHHV, int L, int dtype,
                                 int gate_dtype, int variant, int impl, void* stream) {
  int rc = check_dims(B, NH, S, DHQK, DHHV, L);
  if (rc != MLSTM_OK) return rc;
  if (dtype != MLSTM_F32 && dtype != MLSTM_BF16 && dtype != MLSTM_F16) return MLSTM_ERR_DTYPE;
  if (gate_dtype != MLSTM_F32 && gate_dtype != MLSTM_BF16 && gate_dtype != MLSTM_F16) return MLSTM_ERR_DTYPE;
  if (variant < MLSTM_EXP || variant > MLSTM_SIG_NONORM) return MLSTM_ERR_UNSUPPORTED;
  if (!k || !v || !i || !f || !c_last || !m_last || !g_total || !workspace) return MLSTM_ERR_NULL;
  if (variant != MLSTM_SIG_NONORM && !n_last) return MLSTM_ERR_NULL;
  const void* ptrs[] = {k, v, i, f, c_last, n_last, m_last, g_total, workspace};
  for (const void* p : ptrs) if (p && !aligned16(p)) return MLSTM_ERR_ALIGN;
  bool use_sm100 = false;
  if ((rc = resolve_impl(impl, B, NH, S, DHQK, DHHV, L, dtype, &use_sm100)) != MLSTM_OK) return rc;
  const ChunkwiseDims d = make_dims(B, NH, S, DHQK, DHHV, L, variant, 1e-6f, dtype);
  SumLayout lay = carve_summary(workspace, B * NH, d.SP, d.NC);
  if (workspace_bytes < lay.bytes) return MLSTM_ERR_WORKSPACE;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  // the segment starts from the empty state: C = 0, n = 0, m = -inf
  if ((rc = launch_gates(gate_dtype, i, f, nullptr, nullptr, nullptr, lay.gb, lay.m_states, d, st, -INFINITY, g_total)) != MLSTM_OK) return rc;
  if (use_sm100) {
    if ((rc = sm100_recurrent_fw(k, v, lay.gb, nullptr, nullptr, nullptr, nullptr, c_last, n_last, d, st)) != MLSTM_OK) return rc;
  } else {
    if ((rc = simt_recurrent_fw(dtype, MLSTM_F32, k, v, lay.gb, nullptr, nullptr, nullptr, nullptr, c_last, n_last, d, st)) != MLSTM_OK) return rc;
  }
  MLSTM_CUDA_CHECK(cudaMemcpy2DAsync(m_last, sizeof(float), lay.m_states + d.NC, sizeof(float) * (d.NC + 1),
                                     sizeof(float), (size_t)B * NH, cudaMemcpyDeviceToDevice, st));
  return MLSTM_OK;
}

int mlstm_b200_state_combine(const float* c_in, const float* n_in, const float* m_in, const float* c_loc,
                             const float* n_loc, const float* m_loc, const float* g_total, float* c_out,
                             float* n_out, float* m_out, int B, int NH, int DHQK, int DHHV, int variant,
                             void* stream) {
  if (B <= 0 || NH <= 0 || DHQK <= 0 || DHHV <= 0) return MLSTM_ERR_SHAPE;
  if (variant < MLSTM_EXP || variant > MLSTM_SIG_NONORM) return MLSTM_ERR_UNSUPPORTED;
  if (!c_loc || !g_total || !c_out) return MLSTM_ERR_NULL;
  if (variant == MLSTM_EXP && (!m_loc || !m_out)) return MLSTM_ERR_NULL;
  if (n_out && !n_loc) return MLSTM_ERR_NULL;
  return launch_state_combine(c_in, n_in, m_in, c_loc, n_loc, m_loc, g_total, c_out, n_out, m_out, B * NH, DHQK,
                              DHHV, variant, static_cast<cudaStream_t>(stream));
}

int mlstm_b200_step(const void* q, const void* k, const void* v, const void* i, const void* f, const void* c,
                    const void* n, const void* m, void* h, void* c_new, void* n_new, void* m_new, int B, int NH,
                    int DHQK, int DHHV, int dtype, int gate_dtype, int state_dtype, float eps, void* stream) {
  if (B <= 0 || NH <= 0 || DHQK <= 0 || DHHV <= 0 || DHHV % 4 != 0) return MLSTM_ERR_SHAPE;
  if (!q || !k || !v || !i || !f || !c || !n || !m || !h || !c_new || !n_new || !m_new) return MLSTM_ERR_NULL;
  if (n_new == n || m_new == m) return MLSTM_ERR_UNSUPPORTED;
  const void* ptrs[] = {q, k, v, c, n, h, c_new, n_new};
  for (const void* p : ptrs) if (!aligned16(p)) return MLSTM_ERR_ALIGN;
  if (state_dtype != MLSTM_F32 && state_dtype != MLSTM_BF16) return MLSTM_ERR_DTYPE;
  if (gate_dtype != MLSTM_F32 && gate_dtype != MLSTM_BF16 && gate_dtype != MLSTM_F16) return MLSTM_ERR_DTYPE;
  return launch_step(q, k, v, i, f, c, n, m, h, c_new, n_new, m_new, B, NH, DHQK, DHHV, dtype, gate_dtype, state_dtype, eps,
                     static_cast<cudaStream_t>(stream));
}

int mlstm_b200_step_sequence(const void* q, const void* k, const void* v, const void* i, const void* f,
                             const float* c, const float* n, const float* m, void* h, float* c_new, float* n_new,
                             float* m_new, int B, int NH, int T, int DHQK, int DHHV, int dtype, int gate_dtype,
                             float eps, void* stream) {
  if (B <= 0 || NH <= 0 || T <= 0 || DHQK <= 0 || DHHV <= 0 || DHHV % 4 != 0 || DHQK > 512) return MLSTM_ERR_SHAPE;
  if (!q || !k || !v || !i || !f || !h || !c_new || !n_new || !m_new) return MLSTM_ERR_NULL;
  const void* ptrs[] = {q, k, v, c, h, c_new};
  for (const void* p : ptrs) if (p && !aligned16(p)) return MLSTM_ERR_ALIGN;
  if (gate_dtype != MLSTM_F32 && gate_dtype != MLSTM_BF16 && gate_dtype != MLSTM_F16) return MLSTM_ERR_DTYPE;
  return launch_step_sequence(q, k, v, i, f, c, n, m, h, c_new, n_new, m_new, B, NH, T, DHQK, DHHV, dtype, gate_dtype, eps,
                              static_cast<cudaStream_t>(stream));
}

}  // extern "C"
