// Timeline instrumentation for kernel studies (GEMM, attention); compiles to nothing unless
// Z2H_KERNEL_TRACE is defined. Every role of a few chosen CTAs appends SM clock values to its own
// lane of a device array (one array per translation unit) that a host helper copies out after the
// launch.
#pragma once
#ifdef Z2H_KERNEL_TRACE
constexpr int kTraceLen = 512;
static __device__ long long g_kernel_trace[4][3][kTraceLen];
#define Z2H_TRACE_DECL(role) \
  int trace_n = 0;           \
  const int trace_cta = blockIdx.x == 0 ? 0 : (blockIdx.x == gridDim.x - 1 ? 1 : (blockIdx.x == 37 ? 2 : (blockIdx.x == 100 ? 3 : -1))); \
  constexpr int trace_role = role;
#define Z2H_TRACE()                                                                   \
  do {                                                                                \
    if (trace_cta >= 0 && trace_n < kTraceLen) g_kernel_trace[trace_cta][trace_role][trace_n++] = clock64(); \
  } while (0)
#else
#define Z2H_TRACE_DECL(role)
#define Z2H_TRACE()
#endif
