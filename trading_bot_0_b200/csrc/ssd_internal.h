// Internal interfaces between the translation units of the SSD library.
#pragma once
#include "common.cuh"

namespace ssd {

enum { SSD_STAGE_ALL = SSD_STAGE_LOCAL | SSD_STAGE_FINISH };

// `tc` selects the tensor-core stages where they exist (caller has checked tensor_supported).
int run_forward(const Geo& g, int dtype, bool tc, const SsdFwdPtrs& p, char* ws, const WsLayout& w, cudaStream_t s,
                int stages);
int run_backward(const Geo& g, int dtype, bool tc, const SsdBwdPtrs& p, char* ws, const WsLayout& w, cudaStream_t s,
                 int stages);

// tensor-core (tcgen05) stages, bf16 storage, chunk 128.  `tab` = per-head decay tables written by
// the cumsum kernel, `*_bf` = bf16 copies of the chunk-entry states written by the scan over chunks.
bool tensor_supported(const Geo& g, int dtype, const char** why);
int tensor_chunk_state(const Geo& g, int mode, const void* xdy, long long sb, long long sl, const void* bc,
                       long long bsb, long long bsl, const float* tab, float* out, int* status, cudaStream_t s);
int tensor_state_passing(const Geo& g, float* st, const float* cs, const float* init, float* last, void* st_bf,
                         int reverse, bool write, const float* fwd_prev, const void* fwd_prev_bf, const float* fwd_fin,
                         float* sdot, int* sdot_nw,
                         cudaStream_t s);
// both in one launch where it applies (dstate 64, full pass): fp32 `st` optional, bf16 `st_bf` always
bool tensor_state_fused_applies(const Geo& g);
int tensor_state_fused(const Geo& g, int mode, const void* xdy, long long sb, long long sl, const void* bc, long long bsb,
                       long long bsl, const float* tab, float* st, void* st_bf, const float* init, float* last,
                       const void* fwd_prev_bf, const float* fwd_fin, float* sdot, int* sdot_nw, int* status, cudaStream_t s);
int tensor_chunk_scan(const Geo& g, const SsdFwdPtrs& p, const float* tab, const void* prev_bf, int* status,
                      cudaStream_t s);
int tensor_scan_bwd(const Geo& g, const SsdBwdPtrs& p, const float* tab, const void* prev_bf, void* dypb, float* dcsp,
                    float* ddot, int* status, cudaStream_t s);
int tensor_dx(const Geo& g, const SsdBwdPtrs& p, const void* dyp, bool dy_dense, const float* tab, const void* ds_bf,
              float* ddtd, int* status, cudaStream_t s);
bool tensor_bwd_merged_applies(const Geo& g, const SsdBwdPtrs& p);
int tensor_bwd_merged(const Geo& g, const SsdBwdPtrs& p, const float* tab, const void* prev_bf, const void* ds_bf,
                      float* dcsp, float* ddot, float* ddtd, int* status, cudaStream_t s);
// `hmax` [H + 1] int32 tags written by the cumsum kernel: head h decays beyond SSD_SEP_LOG_RANGE inside some chunk iff
// word [h] equals word [H]
int tensor_dbc(const Geo& g, const SsdBwdPtrs& p, const void* dyp, bool dy_dense, const float* tab, const float* hmax,
               const void* prev_bf, const void* ds_bf, int* status, cudaStream_t s);

// status word of a workspace -> SSD_OK / SSD_ERR_TIMEOUT (message set); the sync reader copies it to the host first
int status_code_to_rc(int32_t code, const char* where);
int read_status_sync(const void* word, void* cuda_stream, int32_t* code_out, const char* where);

int tensor_selftest_wait(int* status, long long max_cycles, cudaStream_t s);
int decode_step(const SsdStepDims& d, const SsdStepPtrs& p, cudaStream_t s);
int reset_rows(float* state, long long row_elems, const long long* idx, long long count, long long streams,
               cudaStream_t s);
int sp_total_logdecay(const Geo& g, const float* cs, float* out, cudaStream_t s);
int sp_prefix_state(const float* gs, const float* gl, int world, int rank, int direction, long long bh,
                    long long elems, const float* init, float* out, cudaStream_t s);

}  // namespace ssd
