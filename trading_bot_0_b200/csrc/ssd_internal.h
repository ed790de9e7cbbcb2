// Internal interfaces between the translation units of the SSD library.
#pragma once
#include "common.cuh"

namespace ssd {

enum { SSD_STAGE_ALL = SSD_STAGE_LOCAL | SSD_STAGE_FINISH };

int simt_forward(const Geo& g, int dtype, const SsdFwdPtrs& p, char* ws, const WsLayout& w, cudaStream_t s,
                 int stages);
int simt_backward(const Geo& g, int dtype, const SsdBwdPtrs& p, char* ws, const WsLayout& w, cudaStream_t s,
                  int stages);

int decode_step(const SsdStepDims& d, const SsdStepPtrs& p, cudaStream_t s);
int reset_rows(float* state, long long row_elems, const long long* idx, long long count, long long streams,
               cudaStream_t s);
int sp_total_logdecay(const Geo& g, const float* cs, float* out, cudaStream_t s);
int sp_prefix_state(const float* gs, const float* gl, int world, int rank, int direction, long long bh,
                    long long elems, const float* init, float* out, cudaStream_t s);

}  // namespace ssd
