// Tuning aids of the GEMM kernels: per-CTA phase stamps and wait-time counters written to GemmParams::prof
// (32 slots per CTA; the pointer is null in normal use and every macro then costs one predicated branch).
// They expect `p` (GemmParams) and `t_cta0` (clock64() at CTA start) in scope.
#pragma once

// Optional phase stamps (SM clock, relative to CTA start) for tuning; p.prof is null in normal use.
#define BGEMM_STAMP(slot)                                                                                            \
    do {                                                                                                             \
        if (p.prof) p.prof[(size_t)((blockIdx.z * gridDim.y + blockIdx.y) * gridDim.x + blockIdx.x) * 32 + (slot)] = \
            ((slot) == 10 || (slot) == 11) ? (long long)globaltimer_ns() : clock64() - t_cta0;                                         \
    } while (0)

// Accumulate the clocks a role spends blocked in one kind of wait (tuning aid, only when p.prof is set).
#define BGEMM_TIMED(acc_var, expr)                      \
    do {                                                \
        const long long tw0__ = p.prof ? clock64() : 0; \
        expr;                                           \
        if (p.prof) acc_var += clock64() - tw0__;       \
    } while (0)
#define BGEMM_PUT(slot, value)                                                                                                \
    do {                                                                                                                      \
        if (p.prof) p.prof[(size_t)((blockIdx.z * gridDim.y + blockIdx.y) * gridDim.x + blockIdx.x) * 32 + (slot)] = (value); \
    } while (0)
