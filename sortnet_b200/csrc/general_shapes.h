// Grouped (G > 1) and spatial (HW > 1) shapes of every operator, built on the 2-D kernels.
//
// The operators' general layout is x [B, G, CIg, HW], w [G, W_COg, W_CIg], y [B, G, COg, HW],
// masks [S, G, CI'g] / [S, G, CO'g] (core/cuda/inf_dist_cuda.cu:112-123,152-171,203 in the
// reference).  Each function here repacks the operands of such a call into G independent
// row-major problems, runs the 2-D entry point on each and scatters the results back; the entry
// points call them when G != 1 or HW != 1.  CO, CI, W_CO and W_CI are totals over the groups
// (W_CI = columns of w times G), as at the exported interface and in the reference's binding
// (core/cuda/norm_dist.cpp:139-143).
#pragma once
#include <cuda_runtime.h>

namespace snb {

int general_inf_forward(const float* x, const float* w, int B, int CO, int CI, int G, int HW, float* y,
                        int* pos, const int* ci, const int* co, int W_CO, int W_CI, cudaStream_t st);
int general_inf_backward(const float* g, const int* pos, int B, int CO, int CI, int G, int HW, float* gx,
                         float* gw, const int* ci, const int* co, int W_CO, int W_CI, cudaStream_t st);
int general_lp_forward(const float* x, const float* w, int B, int CO, int CI, int G, int HW, float* y,
                       float p, const int* ci, const int* co, int W_CO, int W_CI, cudaStream_t st);
int general_lp_backward(const float* g, const float* x, const float* w, const float* y, int B, int CO,
                        int CI, int G, int HW, float* gx, float* gw, float p, const int* ci,
                        const int* co, int W_CO, int W_CI, cudaStream_t st);
int general_bound_forward(const float* xl, const float* xu, const float* w, int B, int CO, int CI, int G,
                          int HW, float* yl, float* yu, int* posl, int* posu, cudaStream_t st);
int general_bound_backward(const float* gl, const float* gu, const int* posl, const int* posu, int B,
                           int CO, int CI, int G, int HW, float* gxl, float* gxu, float* gw,
                           cudaStream_t st);
int general_sort_forward(const float* x, const float* w, int B, int CO, int CI, int G, int HW, float* y,
                         int* pos, float q, int K, cudaStream_t st);
int general_sort_bound_forward(const float* xl, const float* xu, const float* w, int B, int CO, int CI,
                               int G, int HW, float* yl, float* yu, float q, int K, cudaStream_t st);
int general_sort_backward(const float* g, const int* pos, int B, int CO, int CI, int G, int HW, float* gx,
                          float* gw, float q, int K, cudaStream_t st);

}  // namespace snb
