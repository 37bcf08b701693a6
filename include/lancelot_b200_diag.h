/*
 * lancelot_b200 - diagnostics for benchmarks.  NOT part of the drop-in boundary
 * (lancelot_b200.h): nothing a binding of the reference's API needs is declared here, and the
 * reference has no counterpart for any of it.
 */
#ifndef LANCELOT_B200_DIAG_H
#define LANCELOT_B200_DIAG_H

#include "lancelot_b200.h"

#ifdef __cplusplus
extern "C" {
#endif

/* number of kernels this library has launched in this process */
LB_API unsigned long long lb_launch_count(void);

/* Per-kernel device times.  enable != 0 clears the record and starts timing: an event is recorded on the
 * launching stream in front of every kernel the library launches.  lb_diag_kernel_report synchronises,
 * writes a JSON object {"kernel name": {"launches": n, "ms": t}, ...} into buf and clears the record;
 * a kernel's time runs to the next launch on the stream (or to the report), so it includes copies and
 * gaps that follow it.  Meant for one stream at a time; at most 32768 launches per record. */
LB_API int lb_diag_kernel_timing(int enable);
LB_API int lb_diag_kernel_report(char *buf, size_t capacity);

/* Measures the register-only rate of one of the transform's butterfly variants on this GPU (butterflies per
 * second, synchronous, a few milliseconds): the arithmetic ceiling of any NTT schedule for primes of that size.
 * variant: 0 integer Shoup product with conditional subtraction (primes of 58 bits and more), 1 the same without
 * it (below 2^58), 2 the whole butterfly on the FP64 pipe with one centred reduction per element and pass (primes of
 * [2^47, 2^50)), 3 the same at a 40-bit prime (primes below 2^47; the transform kernels skip most of those
 * reductions there), -1 the variant the context's first prime takes.  One limb needs (N/2) log2 N butterflies for
 * its 16 N bytes. */
LB_API int lb_probe_butterfly_rate(lb_context *ctx, int variant, double *butterflies_per_second);

#ifdef __cplusplus
}
#endif
#endif
