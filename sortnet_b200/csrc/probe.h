/* Issue-cost probes (bench / profiling only; not part of the product ABI in include/sortnet_b200.h).
 * The library exports them so that run_case.py can time them; they have no counterpart in the
 * reference. */
#ifndef SORTNET_B200_PROBE_H
#define SORTNET_B200_PROBE_H
#ifdef __cplusplus
extern "C" {
#endif

/* Runs a register-only loop of the max-plus inner step in instruction form `variant` (0..8);
 * *pairs = output-pairs processed, each two reduction steps.
 * scratch: at least 2 * SMs * 256 + 64 floats of device memory, first 64 read as operands. */
int snb_probe_step(int variant, float* scratch, int iters, double* pairs, void* stream);

#ifdef __cplusplus
}
#endif
#endif
