/*
 * ssd_b200.h - C ABI of the B200 (sm_100a) Mamba-2 SSD operator library.
 *
 * Every entry point takes plain pointers and sizes: raw CUDA device pointers (what
 * `at_data_ptr` returns for a tch tensor, vendor/torch-sys-0.25.0/libtch/torch_api.h:41),
 * a caller-owned workspace, and the CUDA stream to launch on.  The library never allocates
 * or frees device memory, never synchronises the host with the device, never changes the
 * current device, and keeps no pointer after a call returns, so every call may be issued
 * while the caller's stream is being captured into a CUDA graph (the PPO update of the
 * reference runs its forward+backward inside one: trading_bots/src/torch/train/update.rs:206-328,
 * vendor/torch-sys-0.25.0/libtch/torch_api.cpp:403-436).
 *
 * Error convention (mirrors libtch's PROTECT / torch_last_err,
 * vendor/torch-sys-0.25.0/libtch/torch_api.h:9,18-23): functions return 0 on success or a
 * negative SsdStatus; a human-readable message is kept per thread and read with
 * ssd_last_error().
 *
 * Operator (per batch b, head h with group g = h*ngroups/nheads, time t, state S [P x N]):
 *     dt[b,t,h] = act(dt_in[b,t,h] + dt_bias[h])   act = softplus if dims.dt_softplus else identity; dt_bias optional
 *     a_t = exp(dt[b,t,h] * A[h])
 *     S_t = a_t * S_{t-1} + dt[b,t,h] * x[b,t,h,:] (outer) B[b,t,g,:]
 *     y_t = S_t . C[b,t,g,:] + D[h] * x[b,t,h,:]          (then y_t *= silu(z_t) if z given)
 */
#ifndef SSD_B200_H
#define SSD_B200_H

#include <stddef.h>
#include <stdint.h>

#if defined(__GNUC__)
#define SSD_API __attribute__((visibility("default")))
#else
#define SSD_API
#endif

#ifdef __cplusplus
extern "C" {
#endif

typedef enum SsdStatus {
  SSD_OK = 0,
  SSD_ERR_BAD_SHAPE = -1,
  SSD_ERR_BAD_ALIGNMENT = -2,
  SSD_ERR_UNSUPPORTED = -3,
  SSD_ERR_WORKSPACE_TOO_SMALL = -4,
  SSD_ERR_CUDA = -5,
  SSD_ERR_NULL_POINTER = -6,
  SSD_ERR_TIMEOUT = -7
} SsdStatus;

typedef enum SsdDtype { SSD_F32 = 0, SSD_BF16 = 1 } SsdDtype;

typedef enum SsdPass { SSD_PASS_FWD = 0, SSD_PASS_BWD = 1 } SsdPass;

/* Kernel family selection.  AUTO picks the tcgen05 tensor-core kernels when dtype is bf16 and
 * the shape is one they cover, else the exact-fp32 CUDA-core kernels.  TENSOR insists on the
 * tensor-core family (an error where it does not apply).  TENSOR_ONETILE is the same family
 * restricted to its one-tile-per-CTA kernels (no persistent pipelines, chunk states and the
 * scan over chunks as two kernels): the comparison arm the persistent kernels are measured
 * against.  The library reads no environment variable; this field is the only switch. */
typedef enum SsdAlgo {
  SSD_ALGO_AUTO = 0, SSD_ALGO_FP32_CORES = 1, SSD_ALGO_TENSOR = 2, SSD_ALGO_TENSOR_ONETILE = 3
} SsdAlgo;

/*
 * Problem geometry.  `dtype` is the storage type of x, dt, B, C, z, y and of dx, dB, dC, dz, dy;
 * A, D, states, ddt, dA, dD are always fp32.  All arithmetic accumulates in fp32.
 * `chunk` (<= 256) is the evaluation schedule only: results do not depend on it.  The tensor-core
 * family evaluates 128-long chunks; a chunk of 256 is run as two of them.
 * Strides are in ELEMENTS for the batch and sequence dims; the remaining dims are dense
 * (x/z/y/dy: [.., H, P]; dt: [.., H]; B/C: [.., G, N]).  A stride of 0 means "dense default".
 * This is how a narrowed / non-contiguous tch view is passed (the reference accepts those on
 * its attention path, trading_bots/src/torch/fa4.rs:283-305).
 */
typedef struct SsdDims {
  int32_t batch, seqlen, nheads, headdim, dstate, ngroups, chunk;
  int32_t dtype;     /* SsdDtype */
  int32_t algo;      /* SsdAlgo  */
  int32_t device;    /* CUDA ordinal the pointers live on; -1 = do not check */
  int32_t has_z;     /* 1 if a z gate is passed (sizes the backward workspace) */
  int32_t dt_softplus; /* 1: the step size is softplus(dt + dt_bias), fused into the cumsum kernel and its backward
                          (the activation a Mamba-2 layer applies just before the scan); 0: dt + dt_bias as given */
  int64_t x_stride_b, x_stride_l;
  int64_t dt_stride_b, dt_stride_l;
  int64_t b_stride_b, b_stride_l;
  int64_t c_stride_b, c_stride_l;
  int64_t z_stride_b, z_stride_l;
  int64_t y_stride_b, y_stride_l;   /* y in forward, dy in backward */
} SsdDims;

/* Forward operands.  Optional pointers may be NULL. */
typedef struct SsdFwdPtrs {
  const void* x;           /* [B,L,H,P]  dtype */
  const void* dt;          /* [B,L,H]    dtype  (positive after the optional bias / softplus) */
  const float* A;          /* [H]        fp32, negative */
  const void* Bm;          /* [B,L,G,N]  dtype */
  const void* Cm;          /* [B,L,G,N]  dtype */
  const float* D;          /* [H]        fp32, optional */
  const void* z;           /* [B,L,H,P]  dtype, optional gate: y *= silu(z) */
  const float* init_state; /* [B,H,P,N]  fp32, optional */
  void* y;                 /* [B,L,H,P]  dtype, out */
  float* final_state;      /* [B,H,P,N]  fp32, out, optional */
  const float* dt_bias;    /* [H]        fp32, optional: added to dt before the activation */
} SsdFwdPtrs;

/* Backward operands: the forward inputs again, the incoming gradients, the outputs. */
typedef struct SsdBwdPtrs {
  const void* x; const void* dt; const float* A; const void* Bm; const void* Cm;
  const float* D; const void* z; const float* init_state;
  const void* dy;            /* [B,L,H,P] dtype: gradient w.r.t. the (gated) output */
  const float* dfinal_state; /* [B,H,P,N] fp32, optional */
  void* dx;                  /* [B,L,H,P] dtype, dense */
  float* ddt;                /* [B,L,H]   fp32,  dense */
  float* dA;                 /* [H]       fp32 */
  void* dB;                  /* [B,L,G,N] dtype, dense */
  void* dC;                  /* [B,L,G,N] dtype, dense */
  float* dD;                 /* [H]       fp32, optional (required iff D given) */
  void* dz;                  /* [B,L,H,P] dtype, dense, required iff z given */
  float* dinit_state;        /* [B,H,P,N] fp32, optional */
  int32_t fwd_saved;         /* 1: `workspace` is the buffer ssd_forward ran in for these same
                                inputs (its chunk cumsums and chunk-entry states are reused);
                                0: recompute them.  The buffer must have had the backward's size
                                (ssd_workspace_bytes(dims, 1)) already when the forward ran: a
                                forward into a forward-sized buffer keeps nothing for a backward. */
  const float* dt_bias;      /* [H] fp32, optional, as in the forward */
  float* ddt_bias;           /* [H] fp32, out, required iff dt_bias given.  With dt_bias / dt_softplus, `ddt` is the
                                gradient w.r.t. the dt that was passed in (before bias and activation). */
} SsdBwdPtrs;

/* Single-timestep recurrence for streamed rollout (in place on `state`). */
typedef struct SsdStepDims {
  int32_t streams, nheads, headdim, dstate, ngroups;
  int32_t dtype;        /* SsdDtype of x, dt, B, C, z, y; state is always fp32 */
  int32_t device;       /* -1 = do not check */
  int32_t dt_softplus;  /* as in SsdDims */
  int64_t x_stride_s;   /* elements between streams; 0 = dense */
  int64_t dt_stride_s, b_stride_s, c_stride_s, z_stride_s, y_stride_s;
} SsdStepDims;

typedef struct SsdStepPtrs {
  float* state;        /* [S,H,P,N] fp32, updated in place */
  const void* x;       /* [S,H,P] */
  const void* dt;      /* [S,H]   */
  const float* A;      /* [H] */
  const void* Bm;      /* [S,G,N] */
  const void* Cm;      /* [S,G,N] */
  const float* D;      /* [H], optional */
  const void* z;       /* [S,H,P], optional */
  void* y;             /* [S,H,P], out */
  const float* dt_bias;/* [H] fp32, optional */
} SsdStepPtrs;

/* Bytes of workspace ssd_forward / ssd_backward need for `dims` (0 on invalid dims, with the
 * error string set).  The backward workspace begins with the forward layout, so one buffer of
 * the backward size serves both calls.  Replaces: nothing in the reference (its SSD layer was
 * removed; only its timings remain, benchmark_results/bench_20260112_070055.json:6-41). */
SSD_API size_t ssd_workspace_bytes(const SsdDims* dims, int32_t pass);

/* y, final_state = SSD(x, dt, A, B, C, D, z, init_state), chunked evaluation.  Sits where the
 * reference's blocks call their sequence mixer today
 * (`Tensor::scaled_dot_product_attention`, trading_bots/src/torch/model/blocks/gqa.rs:95-104;
 * FA4 prefill, trading_bots/src/torch/world_model.rs:1099-1103). */
SSD_API int32_t ssd_forward(const SsdDims* dims, const SsdFwdPtrs* p, void* workspace, size_t workspace_bytes,
                    void* cuda_stream);

/* Gradients of ssd_forward.  The reference never hand-writes a backward (autograd through
 * SDPA / FA4, trading_bots/src/torch/fa4.rs:98-138); tch-rs has no custom autograd node, so the
 * contract is an explicit call. */
SSD_API int32_t ssd_backward(const SsdDims* dims, const SsdBwdPtrs* p, void* workspace, size_t workspace_bytes,
                     void* cuda_stream);

/* One timestep over `streams` independent recurrences, in place on `state`.  Takes the slot of
 * `TradingModel::step_on_device` (trading_bots/src/torch/model/stream/live.rs:257-320) and of
 * the Q=1 decode (trading_bots/src/torch/world_model.rs:1213-1247) in the rollout loop
 * (trading_bots/src/torch/train/rollout.rs:209-235). */
SSD_API int32_t ssd_state_update(const SsdStepDims* dims, const SsdStepPtrs* p, void* cuda_stream);

/* Zero the state rows of the streams listed in `stream_idx` (device int64 indices, `count` of
 * them) without a host sync: the per-environment reset of the reference
 * (trading_bots/src/torch/model/stream/live.rs:114-158, which avoids a sync at :155-157). */
SSD_API int32_t ssd_state_reset_rows(float* state, int64_t row_elems, const int64_t* stream_idx, int64_t count,
                             int64_t streams, void* cuda_stream);

/*
 * Sequence-parallel split.  A rank that owns a contiguous slice of the sequence cannot finish
 * its scan before it knows the state entering the slice, so both passes are exposed in stages:
 *   SSD_STAGE_LOCAL  - per-chunk work that needs no cross-chunk state (cumsum, chunk states;
 *                      in backward also the forward recompute and the local state gradients)
 *   SSD_STAGE_TOTAL  - read-only scan giving the slice total for a ZERO boundary state:
 *                      forward writes it to final_state, backward to dinit_state
 *   SSD_STAGE_FINISH - the scan with the true boundary state (init_state / dfinal_state) and
 *                      everything downstream of it
 * ssd_forward == stages LOCAL|FINISH.  Between TOTAL and FINISH every rank obtains the (total state,
 * total log-decay) records of the ranks before (direction +1) or after (direction -1) it, and
 * ssd_sp_prefix_state folds them:
 *   +1: acc = boundary; for q = 0 .. rank-1:          acc = exp(logdecay_q) * acc + state_q
 *   -1: acc = boundary; for q = world-1 .. rank+1:    acc = exp(logdecay_q) * acc + state_q
 * No counterpart in the reference (it is a single-GPU program with no collective anywhere).
 */
/* SSD_STAGE_LOCAL can be given in two halves so that the exchange overlaps local work that does not need it:
 *   SSD_STAGE_LOCAL_STATES - the part of LOCAL the TOTAL stage needs (backward: the local state gradients; forward: all
 *                            of LOCAL)
 *   SSD_STAGE_LOCAL_REST   - the remainder (backward, ungated: the forward recompute pass that yields the per-position
 *                            row sums and is only read by FINISH; with a z gate the state gradients read what that pass
 *                            writes, so LOCAL_STATES then runs both and LOCAL_REST is empty).  Call it after LOCAL_STATES,
 *                            on any stream ordered after that call and before FINISH. */
enum { SSD_STAGE_LOCAL = 1, SSD_STAGE_TOTAL = 2, SSD_STAGE_FINISH = 4, SSD_STAGE_LOCAL_STATES = 8, SSD_STAGE_LOCAL_REST = 16 };

SSD_API int32_t ssd_forward_staged(const SsdDims* dims, const SsdFwdPtrs* p, void* workspace, size_t workspace_bytes,
                           void* cuda_stream, int32_t stages);
SSD_API int32_t ssd_backward_staged(const SsdDims* dims, const SsdBwdPtrs* p, void* workspace, size_t workspace_bytes,
                            void* cuda_stream, int32_t stages);

/* out[b,h] = sum over this slice of dt*A, read from the chunk cumsums a LOCAL stage left in
 * `workspace`. */
SSD_API int32_t ssd_sp_total_logdecay(const SsdDims* dims, const void* workspace, size_t workspace_bytes, float* out,
                              void* cuda_stream);

/* gathered_states [world, batch_heads, state_elems] fp32, gathered_logdecay [world, batch_heads]
 * fp32, boundary [batch_heads, state_elems] fp32 or NULL (zero), state_in out, same shape. */
SSD_API int32_t ssd_sp_prefix_state(const float* gathered_states, const float* gathered_logdecay, int32_t world,
                            int32_t rank, int32_t direction, int64_t batch_heads, int64_t state_elems,
                            const float* boundary, float* state_in, void* cuda_stream);

/*
 * The exchange itself, for hosts that have no collective library of their own in reach (a Rust / tch program has no
 * torch.distributed): NCCL over NVLink, bound at run time (dlopen of libnccl.so.2; nothing is loaded until the first
 * ssd_sp_* call).  SsdSpComm is an owning handle with a new / free pair, the convention the reference uses for the
 * objects it added to its shim (at_cuda_graph_new / at_cuda_graph_free, vendor/torch-sys-0.25.0/libtch/torch_api.cpp:378-401).
 *   ssd_sp_unique_id   - rank 0 makes the 128-byte NCCL id; the host program hands it to the other ranks by its own means
 *   ssd_sp_comm_new    - collective over all ranks, on the current device; NULL on failure (ssd_last_error)
 *   ssd_sp_comm_wrap   - borrow an ncclComm_t the host already has (not destroyed by ssd_sp_comm_free)
 *   ssd_sp_exchange_fwd / _bwd - after the LOCAL|TOTAL stages: reads the slice's total log-decay from the chunk cumsums in
 *       `workspace`, sends this rank's (slice-total state, log-decay) record to the ranks after (fwd) / before (bwd) it and
 *       receives theirs from the ranks before / after it into `exchange_buf` (LOCAL memory; ssd_sp_exchange_bytes gives its
 *       size; one NCCL group of point-to-point transfers), and folds the received records into `state_in` / `dstate_out`, which then goes to the FINISH stage as init_state / dfinal_state.
 *       `init_state` / `dfinal_state` here are the boundary of the GLOBAL sequence (same on every rank, or NULL).
 *       Everything is enqueued on `cuda_stream`.  timeout_ms == 0: return at once (legal during stream capture).
 *       timeout_ms > 0 (checked mode): a fixed-size signature of the problem goes round first and is compared on the host
 *       (SSD_ERR_BAD_SHAPE names the rank that disagrees), and the call waits for the exchange on the host for at most
 *       that long: SSD_ERR_TIMEOUT when a rank never joined.  After a timeout the communicator is in an unknown state:
 *       ssd_sp_comm_abort, then make a new one.  No kernel of this library and no TMA ever reads a peer's memory.
 *   ssd_sp_allreduce_params - dA (and dD) summed over ranks in place: the parameters are replicated.
 * No counterpart in the reference (single GPU, no collective anywhere).
 */
#define SSD_SP_UNIQUE_ID_BYTES 128
typedef struct SsdSpComm SsdSpComm;
SSD_API int32_t ssd_sp_unique_id(void* id128);
SSD_API SsdSpComm* ssd_sp_comm_new(const void* id128, int32_t world, int32_t rank);
SSD_API SsdSpComm* ssd_sp_comm_wrap(void* nccl_comm);
SSD_API int32_t ssd_sp_comm_world(const SsdSpComm* comm);
SSD_API int32_t ssd_sp_comm_rank(const SsdSpComm* comm);
SSD_API void ssd_sp_comm_free(SsdSpComm* comm);
SSD_API int32_t ssd_sp_comm_abort(SsdSpComm* comm);
SSD_API size_t ssd_sp_exchange_bytes(const SsdDims* dims, int32_t world);
SSD_API int32_t ssd_sp_exchange_fwd(const SsdDims* dims, const void* workspace, size_t workspace_bytes, SsdSpComm* comm,
                                    const float* local_final_state, const float* init_state, float* state_in,
                                    void* exchange_buf, size_t exchange_bytes, void* cuda_stream, int32_t timeout_ms);
SSD_API int32_t ssd_sp_exchange_bwd(const SsdDims* dims, const void* workspace, size_t workspace_bytes, SsdSpComm* comm,
                                    const float* local_dinit_state, const float* dfinal_state, float* dstate_out,
                                    void* exchange_buf, size_t exchange_bytes, void* cuda_stream, int32_t timeout_ms);
SSD_API int32_t ssd_sp_allreduce_params(SsdSpComm* comm, float* dA, float* dD /* optional */, int32_t nheads,
                                        void* cuda_stream, int32_t timeout_ms);

/* Message for the last failing call on this thread ("" if none); valid until the next call on
 * this thread.  Mirrors `get_and_reset_last_err` (trading_bots/src/torch/cuda/graph.rs:107-118). */
SSD_API const char* ssd_last_error(void);

/*
 * Forward pass that allocates nothing and takes no workspace argument: the scratch that
 * ssd_forward gets from its caller comes instead from a fixed SSD_NOALLOC_MAX_BYTES array built
 * into the library (present on every GPU that loads the library, until the process exits).
 * For callers that cannot obtain device memory at the point of the call: a rollout or live
 * trading loop running after its memory pool was frozen, a host that holds raw device pointers
 * from an FFI but no allocator, a process whose free device memory is already committed.
 * The caller still passes every input and output tensor.  Problems whose forward workspace
 * (ssd_workspace_bytes(dims, SSD_PASS_FWD)) exceeds SSD_NOALLOC_MAX_BYTES are rejected with
 * SSD_ERR_WORKSPACE_TOO_SMALL and a message naming both sizes.  The first call on each device
 * looks up the array's device address (make that first call before any stream capture); no
 * call allocates or frees device memory.  Every call on a device shares the one array: calls
 * whose kernels could overlap on the GPU (different streams, or different host threads) race
 * and must be serialised by the caller; the array keeps the previous call's contents and the
 * entry point re-initialises what it needs.  Results equal ssd_forward's for the same inputs.
 * A bounded wait that ran out inside such a call is reported by ssd_noalloc_status (below).
 * This entry point has no counterpart in the reference.
 */
#define SSD_NOALLOC_MAX_BYTES ((size_t)32 << 20)
SSD_API int32_t ssd_forward_noalloc(const SsdDims* dims, const SsdFwdPtrs* p, void* cuda_stream);
SSD_API size_t ssd_noalloc_max_bytes(void);

/*
 * The two bandwidth-bound operators either side of the scan in a Mamba-2 layer (the step-size activation
 * softplus(dt + dt_bias) and the gate y * silu(z) are inside the scan itself, see SsdDims / SsdFwdPtrs):
 *
 *   before: out[b,t,c] = act(bias[c] + sum_k weight[c,k] * in[b, t-width+1+k, c])   causal, depthwise, zero history;
 *           the layer runs it over the concatenated (x | B | C) channels and hands the three channel ranges of `out`
 *           to ssd_forward as strided views.  The reference has the same 3-tap causal depthwise convolution on its
 *           q/k/v (trading_bots/src/torch/model/blocks/gqa.rs:148-178).
 *   after : out[r,:] = in[r,:] * rsqrt(mean(in[r,:]^2) + eps) * weight   over the H*P features of a token; weight is
 *           optional (the reference's RMS norm has no gain, trading_bots/src/torch/model/rmsnorm.rs:16-19).
 *
 * Storage dtype bf16 or fp32, arithmetic fp32; weight, bias, rstd and their gradients fp32.  Strides in ELEMENTS,
 * multiples of 16 bytes; channels / width multiples of 8.  The backward calls recompute what they need from the
 * forward INPUT; the conv backward takes the incoming gradient as up to three channel segments so that the scan's
 * dx, dB, dC tensors are consumed where they lie.  Reductions over tokens use a fixed summation order.
 */
typedef struct SsdConvDims {
  int32_t batch, seqlen, channels, width;   /* width = taps, 2..4 */
  int32_t dtype;                            /* SsdDtype of in, out and their gradients */
  int32_t device;                           /* -1 = do not check */
  int32_t activation;                       /* 0 identity, 1 silu */
  int32_t reserved;
  int64_t in_stride_b, in_stride_l, out_stride_b, out_stride_l;
} SsdConvDims;

typedef struct SsdConvGrad {                /* one channel segment of the gradient w.r.t. `out` */
  const void* ptr;                          /* [B, L, channels] with the strides below */
  int32_t channels, reserved;
  int64_t stride_b, stride_l;
} SsdConvGrad;

typedef struct SsdNormDims {
  int64_t rows;                             /* batch * seqlen */
  int32_t width;                            /* features per row, <= 2048 */
  int32_t dtype, device;
  float eps;
  int64_t in_stride_row, out_stride_row;
} SsdNormDims;

SSD_API size_t ssd_conv1d_workspace_bytes(const SsdConvDims* dims);   /* backward only */
SSD_API int32_t ssd_conv1d_forward(const SsdConvDims* dims, const void* in, const float* weight /* [C,width] */,
                                   const float* bias /* [C], optional */, void* out, void* cuda_stream);
SSD_API int32_t ssd_conv1d_backward(const SsdConvDims* dims, const void* in, const float* weight, const float* bias,
                                    const SsdConvGrad* dout, int32_t ndout, void* din, int64_t din_stride_b,
                                    int64_t din_stride_l, float* dweight, float* dbias /* optional */, void* workspace,
                                    size_t workspace_bytes, void* cuda_stream);
SSD_API size_t ssd_rmsnorm_workspace_bytes(const SsdNormDims* dims);  /* backward with a weight only */
SSD_API int32_t ssd_rmsnorm_forward(const SsdNormDims* dims, const void* in, const float* weight /* optional */, void* out,
                                    float* rstd /* [rows], optional, kept for the backward */, void* cuda_stream);
SSD_API int32_t ssd_rmsnorm_backward(const SsdNormDims* dims, const void* in, const float* weight, const float* rstd,
                                     const void* dout, int64_t dout_stride_row, void* din, int64_t din_stride_row,
                                     float* dweight /* iff weight */, void* workspace, size_t workspace_bytes,
                                     void* cuda_stream);

/*
 * Failure detection.  Every wait inside the pipelined kernels (on a TMA transfer, an MMA completion, another warp role)
 * is bounded: when it runs out the kernel writes a code into the first 4 bytes of the workspace (0 = healthy), skips its
 * remaining waits and returns, and later kernels on the same workspace return at once; the context stays usable.
 * ssd_selftest_bounded_wait exercises that path without touching a pipeline: one warp waits, for at most `max_cycles`
 * clock cycles, on a barrier nothing arrives on, then writes 99 to *device_status (a device int32 the caller zeroed).
 * No counterpart in the reference.
 */
SSD_API int32_t ssd_selftest_bounded_wait(int32_t* device_status, int64_t max_cycles, void* cuda_stream);

/*
 * Reading the status word.  The reference follows every FFI call with an error read
 * (`get_and_reset_last_err`, trading_bots/src/torch/cuda/graph.rs:107-118); the device-side counterpart is this word.
 *   ssd_workspace_status        copies the word of `workspace` to the host on `cuda_stream` and WAITS for the stream
 *                               (so it also covers every call issued on that stream before it); returns SSD_OK, or
 *                               SSD_ERR_TIMEOUT with the wait-site code in ssd_last_error() and in *code_out (optional).
 *                               Not while the stream is being captured.
 *   ssd_workspace_status_async  enqueues the 4-byte copy to `code_dst` (device or pinned host memory) and returns at
 *                               once; legal during stream capture.  Feed the value to ssd_status_check after the
 *                               stream (or graph launch) has completed.
 *   ssd_status_check            maps a status word to SSD_OK / SSD_ERR_TIMEOUT (message set).
 *   ssd_noalloc_status          ssd_workspace_status for the array ssd_forward_noalloc computes in, which the caller
 *                               cannot address.
 */
SSD_API int32_t ssd_workspace_status(const void* workspace, void* cuda_stream, int32_t* code_out);
SSD_API int32_t ssd_workspace_status_async(const void* workspace, int32_t* code_dst, void* cuda_stream);
SSD_API int32_t ssd_status_check(int32_t code);
SSD_API int32_t ssd_noalloc_status(void* cuda_stream, int32_t* code_out);

/*
 * Tracing.  ssd_launch_count: kernels this library has launched in this process (all threads).
 * ssd_profile_begin/end: between the two calls every kernel launched from THIS thread gets a
 * CUDA event recorded behind it on its launch stream; _end synchronises on the last event and
 * returns the number of entries written: newline-separated kernel names into `names` and the
 * matching device durations in milliseconds into `ms`.  Not for use during stream capture.  The
 * reference times at wall-clock granularity only (`Instant` around rollout/update,
 * trading_bots/src/torch/train/rollout.rs:24,237); this is the kernel-level counterpart.
 */
SSD_API int64_t ssd_launch_count(void);
SSD_API int32_t ssd_profile_begin(void* cuda_stream);
SSD_API int32_t ssd_profile_end(char* names, size_t names_bytes, float* ms, int32_t max_entries);

/* Library version and the SM architecture it was compiled for (100 for sm_100a). */
SSD_API int32_t ssd_version(void);
SSD_API int32_t ssd_compiled_arch(void);

#ifdef __cplusplus
}
#endif
#endif /* SSD_B200_H */
