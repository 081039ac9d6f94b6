// Timeline instrumentation for kernel studies; compiles to nothing unless Z2H_GEMM_TRACE is defined.
// Each translation unit that includes this file gets its own device array.
#pragma once
// Every role of a few chosen CTAs appends SM clock values to its own lane of a device array that
// a host helper copies out after the launch.
#ifdef Z2H_GEMM_TRACE
constexpr int kTraceLen = 512;
static __device__ long long g_gemm_trace[4][3][kTraceLen];
#define Z2H_TRACE_DECL(role) \
  int trace_n = 0;           \
  const int trace_cta = blockIdx.x == 0 ? 0 : (blockIdx.x == gridDim.x - 1 ? 1 : (blockIdx.x == 37 ? 2 : (blockIdx.x == 100 ? 3 : -1))); \
  constexpr int trace_role = role;
#define Z2H_TRACE()                                                                   \
  do {                                                                                \
    if (trace_cta >= 0 && trace_n < kTraceLen) g_gemm_trace[trace_cta][trace_role][trace_n++] = clock64(); \
  } while (0)
static __device__ int g_epi_n;
#define Z2H_EPI_MARK()                                            \
  do {                                                            \
    if (blockIdx.x == 0 && threadIdx.x == 64) {                   \
      const int n_ = g_epi_n++;                                   \
      if (n_ < kTraceLen) g_gemm_trace[3][2][n_] = clock64();     \
    }                                                             \
  } while (0)
#else
#define Z2H_TRACE_DECL(role)
#define Z2H_TRACE()
#define Z2H_EPI_MARK()
#endif
