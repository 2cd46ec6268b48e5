/*
 * C ABI of the B200 (sm_100a) mLSTM kernel library, libmlstm_b200.so.
 *
 * Every entry point takes raw DEVICE pointers, sizes and a CUDA stream handle
 * (cudaStream_t passed as void*; NULL = the legacy default stream), enqueues its
 * kernels on that stream and returns without synchronising.  The caller owns all
 * buffers.  Tensors are contiguous row-major with the shapes given below and all
 * pointers must be 16-byte aligned.  Return value: MLSTM_OK (0) on success, a
 * negative MLSTM_ERR_* code otherwise (mlstm_b200_error_string() gives the text).
 * Nothing in this library allocates device memory or touches host copies of the
 * data, and there is no CPU fallback.
 *
 * Each entry point names the interface of NX-AI/mlstm_kernels that it replaces
 * (paths relative to that project's root).
 */
#ifndef MLSTM_B200_H
#define MLSTM_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif
#if defined(__GNUC__)
#pragma GCC visibility push(default)
#endif

/* element types of q, k, v, i, f, h and of the gradients */
enum { MLSTM_F32 = 0, MLSTM_BF16 = 1, MLSTM_F16 = 2 };

/* gate variant: exponential input gate with max-state m (mLSTMexp),
 * sigmoid input gate with denominator max(|n|,1) (mLSTMsig, normalize=True),
 * sigmoid input gate without normaliser (mLSTMsig, normalize=False) */
enum { MLSTM_EXP = 0, MLSTM_SIG = 1, MLSTM_SIG_NONORM = 2 };

/* which implementation to run: AUTO picks the tcgen05/TMA kernels whenever the
 * shape allows and the portable CUDA-core kernels otherwise; SIMT / TCGEN05 force one of them
 * (TCGEN05 returns MLSTM_ERR_UNSUPPORTED for a case it does not cover) */
enum { MLSTM_IMPL_AUTO = 0, MLSTM_IMPL_SIMT = 1, MLSTM_IMPL_TCGEN05 = 2 };

enum {
  MLSTM_OK = 0,
  MLSTM_ERR_SHAPE = -1,      /* unsupported or inconsistent sizes */
  MLSTM_ERR_DTYPE = -2,      /* unsupported element type */
  MLSTM_ERR_NULL = -3,       /* a required pointer is NULL */
  MLSTM_ERR_ALIGN = -4,      /* a pointer is not 16-byte aligned */
  MLSTM_ERR_WORKSPACE = -5,  /* workspace too small */
  MLSTM_ERR_CUDA = -6,       /* a CUDA runtime / driver call failed */
  MLSTM_ERR_UNSUPPORTED = -7 /* requested implementation cannot run this case */
};

int mlstm_b200_version(void);
const char* mlstm_b200_error_string(int code);
/* text of the last CUDA error seen by the calling thread inside this library */
const char* mlstm_b200_last_cuda_error(void);

/* Number of kernels this library has launched in the calling process so far. */
long long mlstm_b200_launch_count(void);

/*
 * Waits for the device to go idle and returns the status word of the tcgen05 kernels: 0, or the
 * code (> 0) of the first bounded wait that ran out (the kernel then stopped and its results are
 * invalid); a negative MLSTM_ERR_* value if the query itself failed.  reset != 0 clears the word.
 */
int mlstm_b200_device_status(int reset);

/*
 * Self-test of the bounded waits: launches one tiny kernel in which a single thread waits, for at most
 * limit_polls polls (1 .. 1,000,000: a few milliseconds), on a barrier that nothing ever signals, gives up and
 * records `code` (> 0) in the status word that mlstm_b200_device_status() returns.  Nothing else happens on the
 * device: no copy is in flight and no tensor memory is held.  Lets a host check that an expired wait is reported
 * and leaves the context usable.  No counterpart in the reference (Triton kernels have no device-side waits).
 */
int mlstm_b200_selftest_wait_expiry(unsigned int limit_polls, int code, void* stream);

/*
 * Per-phase device timing.  After mlstm_b200_profile_enable(1) every phase of the entry points
 * below is bracketed by CUDA events on the launching stream; mlstm_b200_profile_read() waits for
 * them, adds up the elapsed milliseconds and the number of occurrences per phase into arrays of
 * mlstm_b200_profile_phases() elements, and clears the record.  Replaces the torch.profiler hook of
 * the reference's benchmark loop (mlstm_kernels/utils/benchmark/runtime.py:56-60,135-136).
 */
int mlstm_b200_profile_enable(int on);
int mlstm_b200_profile_phases(void);
const char* mlstm_b200_profile_phase_name(int phase);
int mlstm_b200_profile_read(float* total_ms, int* count);

/* NVTX ranges (host-side markers named like the profile phases) around every phase of every call, for timeline
 * profilers; off by default.  Returns the previous setting. */
int mlstm_b200_nvtx_enable(int on);

/* 1 if the tcgen05 path covers this chunkwise case, else 0. */
int mlstm_b200_chunkwise_has_tcgen05(int S, int DHQK, int DHHV, int L, int dtype);

/* Element type (MLSTM_F32, or the 16-bit input type on the tcgen05 path) of the per-chunk C state buffer that
 * mlstm_b200_chunkwise_fw writes and mlstm_b200_chunkwise_bw reads, for the given
 * case and implementation choice. */
int mlstm_b200_chunkwise_state_dtype(int S, int DHQK, int DHHV, int L, int dtype, int impl);

/* Scratch bytes the forward (backward = 0), the backward (backward = 1) or the segment summary
 * (backward = 2) call needs. */
size_t mlstm_b200_chunkwise_workspace_bytes(int B, int NH, int S, int DHQK, int DHHV, int L,
                                            int dtype, int variant, int impl, int backward);

/*
 * Chunkwise forward for mLSTMexp / mLSTMsig.
 * Replaces mlstm_chunkwise_fw (mlstm_kernels/torch/chunkwise/triton_xl_chunk/fw.py:20-136)
 * with its two launches, mlstm_chunkwise__recurrent_fw_C (fw_recurrent.py:13-144) and
 * mlstm_chunkwise__parallel_fw_Hintra (fw_parallel.py:14-136), and the sigmoid-gate twin
 * mlstm_siging_chunkwise_fw (mlstm_kernels/torch/chunkwise/triton_xl_chunk_siging/fw.py:20-140).
 *
 *   q, k        (B,NH,S,DHQK)   dtype          v (B,NH,S,DHHV) dtype     i, f (B,NH,S) gate_dtype
 *   c_initial   (B,NH,DHQK,DHHV) f32, n_initial (B,NH,DHQK) f32, m_initial (B,NH) f32; each may be NULL (= zeros)
 *   h           (B,NH,S,DHHV)   dtype   out
 *   n_out,m_out (B,NH,S)        f32     out: denominator max(|n|,e^-m) and combined max state per token
 *   c_states    (B,NH,NC+1,DHQK,DHHV)   out, element type mlstm_b200_chunkwise_state_dtype(); slot k = state
 *                                        before chunk k, slot NC = final state
 *   n_states    (B,NH,NC+1,DHQK) f32 out,  m_states (B,NH,NC+1) f32 out
 *   c_last,n_last,m_last  f32 copies of the final state (B,NH,DHQK,DHHV),(B,NH,DHQK),(B,NH); each may be NULL
 *   L a power of two >= 16.  S % L == 0 for the portable kernels.  Where the tcgen05 kernels run (bf16 or f16,
 *   L = 128, head dims multiples of 8 up to 512 / 1024) S may be ANY length >= 1: NC = ceil(S / L) and the last chunk is ragged - its
 *   missing tokens are read as zeros and switched off in the gates, no output row past S is written.  This
 *   replaces the host-side zero padding of wrap_chunkwise__pad_zeros and the chunk-size ladder 64/32/16 of
 *   wrap_chunkwise__arbitrary_sequence_length (mlstm_kernels/torch/kernel_wrappers.py:76-171,206-267).
 */
/* Large problems (more recurrence CTAs than SMs) are run as two halves of the (batch, head) units on two streams: the
 * caller's and one the library creates per device on first use, forked and joined with events, so that one half's
 * last, partly filled wave of CTAs overlaps the other half's work.  Legal under stream capture.  on = 0 keeps every
 * launch on the caller's stream; returns the previous setting.  mlstm_b200_chunkwise_fw_static never splits. */
int mlstm_b200_set_unit_split(int on);

int mlstm_b200_chunkwise_fw(const void* q, const void* k, const void* v, const void* i, const void* f,
                            const float* c_initial, const float* n_initial, const float* m_initial,
                            void* h, float* n_out, float* m_out,
                            void* c_states, float* n_states, float* m_states,
                            float* c_last, float* n_last, float* m_last,
                            void* workspace, size_t workspace_bytes,
                            int B, int NH, int S, int DHQK, int DHHV, int L,
                            int dtype, int gate_dtype, int variant, int impl, float eps, void* stream);

/*
 * mlstm_b200_chunkwise_fw for callers that cannot allocate device memory.  No counterpart in the
 * reference (its launchers allocate freely through torch).
 *
 * Meant for hosts where cudaMalloc is not an option once they run: runtimes that give all free GPU
 * memory to their own pool at start-up (a later driver allocation then fails), or loops that forbid
 * allocator calls for latency reasons.  Arguments and results are those of mlstm_b200_chunkwise_fw
 * without `workspace`: the scratch lives in a fixed array of mlstm_b200_static_scratch_bytes() bytes
 * (8 MiB) in device global memory that belongs to the library; every GPU that loads the library holds
 * it until the process exits.  The call itself allocates nothing.
 *   - Limit: the case must need no more scratch than that (roughly B*NH*S <= 400,000); larger cases
 *     are rejected with MLSTM_ERR_WORKSPACE before anything is launched.
 *   - The first call on each device looks up the array's device address (a short host-side set-up,
 *     done with that device current); make that first call before any stream capture begins.  The stream
 *     must belong to the current device (checked; MLSTM_ERR_UNSUPPORTED otherwise).
 *   - The CUDA runtime loads device code and the array itself lazily, on first use, and that loading takes
 *     device memory from the driver.  A host that is about to hand all free memory to its own pool should
 *     therefore call mlstm_b200_static_warmup() (array + gate and tcgen05 forward kernels) or run one small
 *     forward per device and implementation BEFORE it does so; only calls after that are free of driver
 *     allocations.  A cudaDeviceReset() invalidates the looked-up address: do not reset a device in use.
 *   - All calls on a device share the one array, which keeps whatever the previous call left in it.
 *     The forward overwrites every word it later reads, so nothing needs clearing; but two calls
 *     whose kernels overlap on the GPU (different streams, or threads) race on it - serialise them.
 */
size_t mlstm_b200_static_scratch_bytes(void);
int mlstm_b200_static_warmup(void);
int mlstm_b200_chunkwise_fw_static(const void* q, const void* k, const void* v, const void* i, const void* f,
                                   const float* c_initial, const float* n_initial, const float* m_initial,
                                   void* h, float* n_out, float* m_out,
                                   void* c_states, float* n_states, float* m_states,
                                   float* c_last, float* n_last, float* m_last,
                                   int B, int NH, int S, int DHQK, int DHHV, int L,
                                   int dtype, int gate_dtype, int variant, int impl, float eps, void* stream);

/*
 * Chunkwise backward (the hand-derived one that ignores the gradient through the
 * denominator).  Replaces mlstm_chunkwise_bw
 * (mlstm_kernels/torch/chunkwise/triton_xl_chunk/bw.py:27-227: bw_recurrent.py:13-120,
 * bw_parallel_dV.py, bw_parallel_dK.py, bw_parallel_dQ.py, chunkwise_gates.py:68-95) and
 * mlstm_siging_chunkwise_bw (mlstm_kernels/torch/chunkwise/triton_xl_chunk_siging/bw.py).
 *
 *   q,k,v,i,f, m_initial as in the forward; c_states, n_out as written by the forward
 *   dh        (B,NH,S,DHHV) dtype;  dc_last (B,NH,DHQK,DHHV) f32 or NULL
 *   dq,dk (B,NH,S,DHQK) dtype out;  dv (B,NH,S,DHHV) dtype out;  di,df (B,NH,S) f32 out
 *   dc_initial (B,NH,DHQK,DHHV) f32 out or NULL
 */
int mlstm_b200_chunkwise_bw(const void* q, const void* k, const void* v, const void* i, const void* f,
                            const float* m_initial, const void* c_states, const float* n_out,
                            const void* dh, const float* dc_last,
                            void* dq, void* dk, void* dv, float* di, float* df, float* dc_initial,
                            void* workspace, size_t workspace_bytes,
                            int B, int NH, int S, int DHQK, int DHHV, int L,
                            int dtype, int gate_dtype, int variant, int impl, float eps, void* stream);

/*
 * Same as mlstm_b200_chunkwise_bw when the forward call of the same problem has just run and its scratch buffer
 * `fw_workspace` (and its m_out output) are still intact: the gate pre-pass (logsigmoid, cumulative sums, max-state
 * recursion) is not repeated, its per-token vectors are read back from that buffer.  The reference keeps no such
 * cache (it recomputes vecB / vecA in mlstm_kernels/torch/chunkwise/triton_xl_chunk/bw.py:116-118).
 * m_out is not read (the buffer holds its own copy of the per-token max state); it may be NULL.
 */
int mlstm_b200_chunkwise_bw_cached(const void* q, const void* k, const void* v, const void* i, const void* f,
                                   const float* m_initial, const void* c_states, const float* n_out,
                                   const float* m_out, const void* fw_workspace, size_t fw_workspace_bytes,
                                   const void* dh, const float* dc_last,
                                   void* dq, void* dk, void* dv, float* di, float* df, float* dc_initial,
                                   void* workspace, size_t workspace_bytes,
                                   int B, int NH, int S, int DHQK, int DHHV, int L,
                                   int dtype, int gate_dtype, int variant, int impl, float eps, void* stream);

/*
 * Per-chunk C states only (no H, no n): what the backward needs when the forward did not keep them.
 * Replaces the state recomputation at the top of the reference's backward when recompute_states_in_bw is set
 * (mlstm_kernels/torch/chunkwise/triton_xl_chunk/bw.py:76-112; switch in fwbw.py:45,62,88-115).
 *   c_states (B,NH,NC+1,DHQK,DHHV) out, element type mlstm_b200_chunkwise_state_dtype().
 *   fw_workspace: the scratch buffer the forward call of the same problem left behind (its gate vectors are read
 *   instead of being recomputed), or NULL - then `workspace` of
 *   mlstm_b200_chunkwise_workspace_bytes(..., backward = 2) bytes is used for a fresh gate pre-pass.
 */
int mlstm_b200_chunkwise_states(const void* k, const void* v, const void* i, const void* f,
                                const float* c_initial, const float* m_initial, void* c_states,
                                const void* fw_workspace, size_t fw_workspace_bytes,
                                void* workspace, size_t workspace_bytes,
                                int B, int NH, int S, int DHQK, int DHHV, int L,
                                int dtype, int gate_dtype, int variant, int impl, void* stream);

/* Backward for a forward that did not keep its per-chunk states (the reference's recompute_states_in_bw = True,
 * mlstm_kernels/torch/chunkwise/triton_xl_chunk/bw.py:76-112): as mlstm_b200_chunkwise_bw_cached, but `c_states_scratch`
 * (same size and element type as the forward's c_states) arrives unwritten and the forward's recurrence is run again, from
 * `c_initial` (f32 or NULL) and the forward's gate vectors, inside the backward's own chains of launches - so that
 * its last wave of CTAs overlaps the state-gradient recurrence instead of standing alone in front of the call. */
int mlstm_b200_chunkwise_bw_recompute(const void* q, const void* k, const void* v, const void* i, const void* f,
                                      const float* m_initial, const float* c_initial, void* c_states_scratch,
                                      const float* n_out, const float* m_out,
                                      const void* fw_workspace, size_t fw_workspace_bytes,
                                      const void* dh, const float* dc_last,
                                      void* dq, void* dk, void* dv, float* di, float* df, float* dc_initial,
                                      void* workspace, size_t workspace_bytes,
                                      int B, int NH, int S, int DHQK, int DHHV, int L,
                                      int dtype, int gate_dtype, int variant, int impl, float eps, void* stream);

/*
 * Sequence-parallel prefill: a long sequence is split into contiguous segments, one per GPU.
 * The reference has no multi-device code; these two entry points implement its state-passing
 * contract (chaining segments through c_initial / n_initial / m_initial and the returned last
 * states: tests/torch/conftest.py:82-175, mlstm_kernels/torch/kernel_wrappers.py:109-151) so that
 * the segments' recurrences can run concurrently.
 *
 * mlstm_b200_chunkwise_summary: gates + inter-chunk recurrence of ONE segment started from the
 *   empty state (C = 0, n = 0, m = -inf).  Outputs the segment's contribution c_last, n_last
 *   (n_last may be NULL for MLSTM_SIG_NONORM), m_last (B,NH) and g_total (B,NH) = sum of
 *   logsigmoid(f) over the segment.  No per-chunk states, no H.
 * mlstm_b200_state_combine: joins the state entering a segment with that segment's summary,
 *   m_out = max(g_total + m_in, m_loc), X_out = exp(g_total + m_in - m_out) X_in + exp(m_loc - m_out) X_loc
 *   (m terms are zero for the sigmoid input gate).  c_in / n_in / m_in may be NULL (zero state, m = 0).
 *   The result equals what the single-device recurrence holds at the segment's end
 *   (mlstm_kernels/triton/chunkwise/xl_chunk/fw_kernel_recurrent.py:175-196 applied per segment).
 * mlstm_b200_chunkwise_dc_summary: the backward twin of the summary.  The state-gradient recurrence of ONE segment
 *   started from a zero incoming gradient: dc_initial (B,NH,DHQK,DHHV) f32 = the segment's own contribution to the
 *   gradient of the state that entered it.  The recurrence is linear, so with dC_right the gradient of the state the
 *   segment handed on,  dC_left = exp(G + m_in - m_out) dC_right + dc_initial  (G, m_in, m_out: total log forget
 *   gate and max state at the two ends of the segment; exp(G) for the sigmoid input gate).  Needs the forward's
 *   scratch buffer (gate vectors) and n_out; `workspace` of B*NH*ceil(S/L)*L floats.  No per-chunk states are written.
 */
int mlstm_b200_chunkwise_summary(const void* k, const void* v, const void* i, const void* f,
                                 float* c_last, float* n_last, float* m_last, float* g_total,
                                 void* workspace, size_t workspace_bytes,
                                 int B, int NH, int S, int DHQK, int DHHV, int L,
                                 int dtype, int gate_dtype, int variant, int impl, void* stream);
int mlstm_b200_state_combine(const float* c_in, const float* n_in, const float* m_in,
                             const float* c_loc, const float* n_loc, const float* m_loc, const float* g_total,
                             float* c_out, float* n_out, float* m_out,
                             int B, int NH, int DHQK, int DHHV, int variant, void* stream);
int mlstm_b200_chunkwise_dc_summary(const void* q, const void* dh, const float* n_out,
                                    const void* fw_workspace, size_t fw_workspace_bytes,
                                    float* dc_initial, void* workspace, size_t workspace_bytes,
                                    int B, int NH, int S, int DHQK, int DHHV, int L,
                                    int dtype, int variant, int impl, float eps, void* stream);

/*
 * One recurrent decode step.  Replaces mlstm_recurrent_step__triton_fw
 * (mlstm_kernels/torch/recurrent/triton_step.py:15-127) and its kernel
 * recurrent_step_fw_kernel (mlstm_kernels/triton/recurrent/fw_step_fused.py:19-195).
 *
 *   q,k (B,NH,DHQK) dtype; v (B,NH,DHHV) dtype; i,f (B,NH) gate_dtype (widened to f32 before any
 *   arithmetic, as fw_step_fused.py:88-94 does)
 *   c (B,NH,DHQK,DHHV), n (B,NH,DHQK), m (B,NH) in state_dtype (MLSTM_F32 or MLSTM_BF16)
 *   h (B,NH,DHHV) dtype out; c_new, n_new, m_new out, state_dtype.
 *   c_new may alias c (each element is read and written by the same thread); n_new and
 *   m_new must not alias n and m.  DHHV % 4 == 0.
 */
int mlstm_b200_step(const void* q, const void* k, const void* v, const void* i, const void* f,
                    const void* c, const void* n, const void* m,
                    void* h, void* c_new, void* n_new, void* m_new,
                    int B, int NH, int DHQK, int DHHV, int dtype, int gate_dtype, int state_dtype, float eps,
                    void* stream);

/*
 * T decode steps in one launch with the state kept on chip between tokens.
 * Replaces the per-token Python loop _mlstm_recurrent_sequence_loop_fw
 * (mlstm_kernels/torch/recurrent/native_sequence.py:13-122) over the step kernel.
 *   q,k (B,NH,T,DHQK); v (B,NH,T,DHHV); i,f (B,NH,T) gate_dtype; h (B,NH,T,DHHV); states f32 as in mlstm_b200_step.
 */
int mlstm_b200_step_sequence(const void* q, const void* k, const void* v, const void* i, const void* f,
                             const float* c, const float* n, const float* m,
                             void* h, float* c_new, float* n_new, float* m_new,
                             int B, int NH, int T, int DHQK, int DHHV, int dtype, int gate_dtype, float eps,
                             void* stream);

#if defined(__GNUC__)
#pragma GCC visibility pop
#endif
#ifdef __cplusplus
}
#endif
#endif /* MLSTM_B200_H */
