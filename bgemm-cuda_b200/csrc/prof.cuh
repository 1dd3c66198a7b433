// Tuning aids of the GEMM kernels: per-CTA phase stamps and wait-time counters written to GemmParams::prof
// (32 slots per CTA). They exist only in builds with -DBGEMM_TUNING; in the default build every macro below
// expands to nothing (BGEMM_TIMED to the bare expression), so the issuer and unpack loops carry no trace of them.
// They expect `p` (GemmParams) and `t_cta0` (clock64() at CTA start) in scope.
#pragma once

#ifdef BGEMM_TUNING

#define BGEMM_TUNING_ONLY(...) __VA_ARGS__
// Phase stamp (SM clock relative to CTA start; slots 10 and 11 take the global timer).
#define BGEMM_STAMP(slot)                                                                                            \
    do {                                                                                                             \
        if (p.prof) p.prof[(size_t)((blockIdx.z * gridDim.y + blockIdx.y) * gridDim.x + blockIdx.x) * 32 + (slot)] = \
            ((slot) == 10 || (slot) == 11) ? (long long)globaltimer_ns() : clock64() - t_cta0;                       \
    } while (0)

// Accumulate the clocks a role spends blocked in one kind of wait.
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
// Event trace of CTA 0 (behind the per-CTA slots of the profile buffer): event `ev`, occurrence `idx`.
#define BGEMM_TRACE(ev, idx)                                                                                        \
    do {                                                                                                            \
        if (p.prof && blockIdx.x == 0 && (idx) < 1024) p.prof[(size_t)gridDim.x * 32 + (ev) * 1024 + (idx)] = clock64() - t_cta0; \
    } while (0)

#else

#define BGEMM_TUNING_ONLY(...)
#define BGEMM_STAMP(slot) do { } while (0)
#define BGEMM_TIMED(acc_var, expr) do { expr; } while (0)
#define BGEMM_PUT(slot, value) do { } while (0)
#define BGEMM_TRACE(ev, idx) do { } while (0)

#endif
