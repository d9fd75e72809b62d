// The grouped fp8 GEMM once more, with its profiling aids compiled in: per-role wait totals,
// SM-clock stamps per tile and per K block, and removal of pipeline stages (wrong results).
// Entry point grouped_fp8_gemm_profiled(); used by benchmarks/bench_grouped_gemm.py only.
#define PPLX_GEMM_PROFILE 1
#include "grouped_gemm.cu"
