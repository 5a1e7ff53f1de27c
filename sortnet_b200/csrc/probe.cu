// Hardware probes: register-only loops that measure what the CUDA cores of the GPU in use can
// sustain.  They have no counterpart in the reference.  The benchmark times them with CUDA
// events to obtain (a) the FP32 FMA peak that its roofline fractions are quoted against and
// (b) the cost of the max-plus inner step in each of its possible instruction forms, which is
// the evidence for the kernel design: on sm_100a every form of "subtract + |.|-max" costs two
// issue cycles per element per scheduler, so 64 elements / clock / SM is the ceiling.
#include "common.cuh"
#include "launch.h"

namespace snb {

__global__ void __launch_bounds__(256) fp32_probe_kernel(float* out, int iters, float a, float b) {
    float acc[16];
#pragma unroll
    for (int i = 0; i < 16; i++) acc[i] = (float)(threadIdx.x + i);
    for (int it = 0; it < iters; it++) {
#pragma unroll
        for (int i = 0; i < 16; i++) acc[i] = fmaf(acc[i], a, b);
    }
    float s = 0.f;
#pragma unroll
    for (int i = 0; i < 16; i++) s += acc[i];
    if (s == 123.456f) out[0] = s;  // never true; keeps the chain alive
}

// One loop iteration = 64 "pairs" (two reduction steps of one output each) per thread
// (32 for the interval-bound variant, which carries two accumulators per output).
template <int V>
__global__ void __launch_bounds__(256) step_probe_kernel(const float* in, float* out, int iters) {
    float acc[8][8], accl[8][8];
    uint64_t xf[8], wf[8];
#pragma unroll
    for (int i = 0; i < 8; i++) {
        xf[i] = pack2(in[threadIdx.x + i], in[threadIdx.x + i + 8]);
        wf[i] = pack2(in[threadIdx.x + i + 16], in[threadIdx.x + i + 24]);
#pragma unroll
        for (int j = 0; j < 8; j++) {
            acc[i][j] = SNB_EPS;
            accl[i][j] = -SNB_EPS;
        }
    }
    const uint64_t delta = pack2(in[0], in[1]);
    for (int it = 0; it < iters; it++) {
#pragma unroll
        for (int i = 0; i < 8; i++) {
#pragma unroll
            for (int j = 0; j < 8; j++) {
                float a, b, c, d, xa, xb, wa, wb;
                unpack2(xf[i], xa, xb);
                unpack2(wf[j], wa, wb);
                if (V == 0) {  // packed subtract + three-input |.|-max
                    unpack2(sub2(xf[i], wf[j]), a, b);
                    acc[i][j] = max3abs(acc[i][j], a, b);
                } else if (V == 1) {  // two scalar subtracts + two two-input max
                    acc[i][j] = fmaxf(acc[i][j], fabsf(xa - wa));
                    acc[i][j] = fmaxf(acc[i][j], fabsf(xb - wb));
                } else if (V == 2) {  // two scalar subtracts + three-input max
                    acc[i][j] = max3abs(acc[i][j], xa - wa, xb - wb);
                } else if (V == 3) {  // packed subtract + two two-input max
                    unpack2(sub2(xf[i], wf[j]), a, b);
                    acc[i][j] = fmaxf(fmaxf(acc[i][j], fabsf(a)), fabsf(b));
                } else if (V == 4) {  // three-input max alone
                    acc[i][j] = max3abs(acc[i][j], xa, wb);
                } else if (V == 5) {  // interval-bound step: 2 scalar subtracts, min3, max3 per element
                    if (i < 4) {      // 32 outputs x 2 accumulators keep the probe in registers
                        float t1 = wa - xa, t2 = xb - wa;
                        accl[i][j] = min3(accl[i][j], t1, t2);
                        acc[i][j] = max3(acc[i][j], t1, t2);
                        t1 = wb - xb;
                        t2 = xa - wb;
                        accl[i][j] = min3(accl[i][j], t1, t2);
                        acc[i][j] = max3(acc[i][j], t1, t2);
                    }
                } else if (V == 6) {  // p = 8 step: packed subtract, two packed squarings, packed fma
                    const uint64_t t = sub2(xf[i], wf[j]);
                    const uint64_t t2 = mul2(t, t), t4 = mul2(t2, t2);
                    unpack2(fma2(t4, t4, pack2(acc[i][j], accl[i][j])), acc[i][j], accl[i][j]);
                } else if (V == 7) {  // two scalar subtracts, sign bits cleared, integer three-input max
                    // (non-negative floats order like their bit patterns)
                    const int ia = __float_as_int(xa - wa) & 0x7fffffff, ib = __float_as_int(xb - wb) & 0x7fffffff;
                    acc[i][j] = __int_as_float(__vimax3_s32(__float_as_int(acc[i][j]), ia, ib));
                } else if (V == 8) {  // integer three-input max alone
                    acc[i][j] = __int_as_float(__vimax3_s32(__float_as_int(acc[i][j]), __float_as_int(xa),
                                                            __float_as_int(wb)));
                }
            }
        }
#pragma unroll
        for (int i = 0; i < 8; i++) xf[i] = sub2(xf[i], delta);
    }
    float s = 0.f;
#pragma unroll
    for (int i = 0; i < 8; i++)
#pragma unroll
        for (int j = 0; j < 8; j++) s += acc[i][j] + accl[i][j];
    out[blockIdx.x * blockDim.x + threadIdx.x] = s;
}

}  // namespace snb

using namespace snb;

// Launches the FMA probe; *flops receives the number of floating-point operations it performs.
extern "C" int snb_probe_fp32(float* scratch, int iters, double* flops, void* stream) {
    if (!scratch || !flops || iters <= 0) return SNB_ERR_NULL_POINTER;
    const int blocks = sm_count() * 8;
    fp32_probe_kernel<<<blocks, 256, 0, (cudaStream_t)stream>>>(scratch, iters, 1.000001f, 1e-7f);
    SNB_CUDA(cudaGetLastError());
    *flops = 2.0 * 16.0 * (double)iters * 256.0 * (double)blocks;
    return SNB_OK;
}

// Launches inner-step probe `variant` (0..8, see step_probe_kernel); *pairs receives the number
// of output-pairs processed (each pair = two reduction steps).  scratch: >= 2 * SMs * 256 + 64
// floats, its first 64 floats are read as operands.
extern "C" int snb_probe_step(int variant, float* scratch, int iters, double* pairs, void* stream) {
    if (!scratch || !pairs || iters <= 0) return SNB_ERR_NULL_POINTER;
    const int blocks = sm_count() * 2;
    cudaStream_t st = (cudaStream_t)stream;
    float* out = scratch + 64;
    switch (variant) {
        case 0: step_probe_kernel<0><<<blocks, 256, 0, st>>>(scratch, out, iters); break;
        case 1: step_probe_kernel<1><<<blocks, 256, 0, st>>>(scratch, out, iters); break;
        case 2: step_probe_kernel<2><<<blocks, 256, 0, st>>>(scratch, out, iters); break;
        case 3: step_probe_kernel<3><<<blocks, 256, 0, st>>>(scratch, out, iters); break;
        case 4: step_probe_kernel<4><<<blocks, 256, 0, st>>>(scratch, out, iters); break;
        case 5: step_probe_kernel<5><<<blocks, 256, 0, st>>>(scratch, out, iters); break;
        case 6: step_probe_kernel<6><<<blocks, 256, 0, st>>>(scratch, out, iters); break;
        case 7: step_probe_kernel<7><<<blocks, 256, 0, st>>>(scratch, out, iters); break;
        case 8: step_probe_kernel<8><<<blocks, 256, 0, st>>>(scratch, out, iters); break;
        default: return SNB_ERR_UNSUPPORTED;
    }
    SNB_CUDA(cudaGetLastError());
    *pairs = (variant == 5 ? 32.0 : 64.0) * (double)iters * 256.0 * (double)blocks;
    return SNB_OK;
}
